"""The multi-process plumbing of bench.py on CPU: two gloo ranks agree on the slowest rank's time and on
the aggregate rate of independent lanes."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_gloo_ranks_take_the_slowest_time():
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        from splash_b200.dist import Group
        g = Group(backend="gloo")
        g.barrier()
        t = 2.0 if g.rank == 0 else 5.0      # seconds each rank measured
        assert g.reduce_max(t) == 5.0
        rate = g.aggregate_rate(16 * 10, t)   # 10 steps of 16 tokens per rank
        assert abs(rate - 2 * 160 / 5.0) < 1e-9, rate
        g.barrier()
        g.close()
        print("rank", g.rank, "ok")
    """ % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, "-c", code], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "rank 0 ok" in outs[0] and "rank 1 ok" in outs[1]
