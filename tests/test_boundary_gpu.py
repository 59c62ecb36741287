"""The drop-in boundary's buffer, event and submission rules on a device (through the C ABI): views keep their base
alive and are checked against its extent, completion can be polled and waited for with a limit, and a second command is
refused while the first one's ticket is out (the reference's MetalBackend rules, runtime/metal/MetalBackend.hpp:42-78,
371-375, 468-478)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
_P = ctypes.c_void_p


def _lib():
    from splash_b200 import lib
    lib.init(0)
    l = lib.load()
    l.sb_view.argtypes = [_P, ctypes.c_size_t, ctypes.c_size_t, ctypes.POINTER(_P)]
    l.sb_event_create.argtypes = [ctypes.POINTER(_P)]
    l.sb_event_query.argtypes = [_P, ctypes.POINTER(ctypes.c_int)]
    l.sb_event_wait_bounded.argtypes = [_P, ctypes.c_uint32]
    l.sb_submit.argtypes = [_P, _P, ctypes.POINTER(ctypes.c_uint64)]
    l.sb_ticket_wait.argtypes = [ctypes.c_uint64, ctypes.c_uint32]
    return lib, l


def test_views_are_checked_and_keep_their_base_alive():
    lib, l = _lib()
    base = _P()
    lib.check(l.sb_alloc(4096, ctypes.byref(base)))
    v1, v2, bad = _P(), _P(), _P()
    lib.check(l.sb_view(base, 1024, 1024, ctypes.byref(v1)))
    assert v1.value == base.value + 1024
    lib.check(l.sb_view(v1, 512, 512, ctypes.byref(v2)))          # a view of a view, inside the same allocation
    assert v2.value == base.value + 1536
    assert l.sb_view(base, 4000, 200, ctypes.byref(bad)) == -1    # past the end: nothing handed out
    assert l.sb_view(v1, 3072, 1, ctypes.byref(bad)) == -1
    assert l.sb_view(ctypes.c_void_p(base.value + (1 << 30)), 0, 16, ctypes.byref(bad)) == -1   # not ours
    lib.check(l.sb_free(base))                                    # the allocation's own hold goes; the views keep it alive
    data = np.arange(256, dtype=np.uint32)
    lib.check(l.sb_upload(v1, data.ctypes.data_as(_P), data.nbytes, None))
    back = np.zeros_like(data)
    lib.check(l.sb_download(back.ctypes.data_as(_P), v1, data.nbytes, None))
    lib.stream_sync()
    assert np.array_equal(back, data)
    lib.check(l.sb_free(v2))
    lib.check(l.sb_free(v1))                                      # the last holder: the memory goes back
    assert l.sb_free(v1) == -1                                    # and the view is no longer known


def test_event_query_and_bounded_wait():
    lib, l = _lib()
    stream = lib.stream_create()
    ev = lib.Event()
    buf = lib.DeviceBuffer(1 << 20)
    lib.check(l.sb_memset(buf.ptr, 0, buf.nbytes, stream))
    ev.record(stream)
    lib.check(l.sb_event_wait_bounded(ev.ptr, 5000))
    done = ctypes.c_int(0)
    lib.check(l.sb_event_query(ev.ptr, ctypes.byref(done)))
    assert done.value == 1


def test_one_command_in_flight():
    """sb_submit hands out a ticket and refuses the next command until sb_ticket_wait has consumed it."""
    lib, l = _lib()
    stream = lib.stream_create()
    buf = lib.DeviceBuffer(64 << 20)
    lib.check(l.sb_graph_begin(stream))
    for i in range(8):
        lib.check(l.sb_memset(buf.ptr, i, buf.nbytes, stream))
    graph = _P()
    lib.check(l.sb_graph_end(stream, ctypes.byref(graph)))
    t1, t2 = ctypes.c_uint64(0), ctypes.c_uint64(0)
    lib.check(l.sb_submit(graph, stream, ctypes.byref(t1)))
    assert l.sb_submit(graph, stream, ctypes.byref(t2)) == -6     # SB_ERR_BUSY: the first ticket is still out
    assert b"in flight" in l.sb_last_error()
    assert l.sb_ticket_wait(t1.value + 1, 10) == -1               # not the command in flight
    lib.check(l.sb_ticket_wait(t1.value, 10000))
    lib.check(l.sb_submit(graph, stream, ctypes.byref(t2)))       # consumed: the next command goes
    assert t2.value == t1.value + 1
    lib.check(l.sb_ticket_wait(t2.value, 10000))
    assert buf.to_numpy(np.uint8, (16,)).tolist() == [7] * 16
    lib.check(l.sb_graph_destroy(graph))
