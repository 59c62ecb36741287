/* splash_b200 - C ABI of the B200-native DFlash2 verify-step kernels.
 *
 * This is the device boundary the host operator layer (splash_b200/csrc/ops/, mirroring the
 * reference's runtime/ops classes) calls in place of the reference's
 * splash::metal::MetalBackend + CommandGraph seam (runtime/metal/MetalBackend.hpp:375-547,
 * runtime/metal/CommandGraph.hpp:26-146): plain pointers and sizes, no C++ or framework types.
 *
 * Conventions
 *  - Every function returns SB_OK (0) or a negative SbStatus; sb_last_error() gives the message of
 *    the calling thread's last failure. Argument and extent errors are reported before anything is
 *    enqueued (the reference throws std::invalid_argument at the same point,
 *    runtime/ops/BufferExtent.hpp:19-27, runtime/ops/Linear.cpp:239-270).
 *  - Pointers named *_dev are device pointers obtained from sb_alloc; streams are opaque handles
 *    from sb_stream_create (0 = the default stream).
 *  - Kernels never trap: a device-side contract violation or an expired bounded wait sets the
 *    context's status word, read with sb_device_status() (mirrors
 *    runtime/metal/kernels/common/attention_sequence.h:28-34).
 *  - There is no CPU fallback: every compute entry point fails with SB_ERR_NO_DEVICE without a GPU.
 */
#ifndef SPLASH_B200_H
#define SPLASH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_API __attribute__((visibility("default")))

typedef enum SbStatus {
  SB_OK = 0,
  SB_ERR_INVALID = -1,   /* bad argument or buffer extent; nothing was enqueued */
  SB_ERR_NO_DEVICE = -2, /* no CUDA device / sb_init not called */
  SB_ERR_CUDA = -3,      /* a CUDA runtime call failed */
  SB_ERR_OOM = -4,       /* allocation refused (runtime/metal/Allocation.hpp:16-31: a value, not a crash) */
  SB_ERR_DEVICE = -5,    /* the device status word is set */
  SB_ERR_BUSY = -6       /* a command is still in flight (runtime/metal/MetalBackend.hpp:371-375) */
} SbStatus;

/* Weight formats: the ids of the reference's quant format table (runtime/metal/abi/QuantFormat.h:79-124). */
enum {
  SB_FMT_Q4K = 0,
  SB_FMT_Q6K = 4,
  SB_FMT_Q80 = 6,
  SB_FMT_NVFP4 = 37,
  SB_FMT_BF16 = 41,
  SB_FMT_F16 = 42,
  SB_FMT_F32 = 64 /* plain fp32 rows (GDN alpha/beta, MoE router: runtime/ops/LinearGguf.cpp:559-604) */
};

/* Epilogues of a projection (runtime/ops/Linear.hpp:73, runtime/metal/kernels/common/gguf_tile.h:8-14). */
enum {
  SB_EPILOGUE_NONE = 0,
  SB_EPILOGUE_RESIDUAL = 1,     /* out = v + aux */
  SB_EPILOGUE_UP_WITH_GATE = 2, /* out = bf16(v) * silu(aux) */
  SB_EPILOGUE_GATE_UP = 3       /* one pass over gate and up rows: bf16(bf16(up) * silu(bf16(gate))) */
};

/* ---- context, memory, streams, events (replaces MetalBackend's buffer and command API) ---- */

SB_API int sb_device_count(void);
SB_API int sb_init(int device);
SB_API const char *sb_last_error(void);
/* Reads and clears the device status word (0 = healthy). Synchronizes the device. */
SB_API int sb_device_status(uint32_t *status);
SB_API int sb_sm_count(void);

SB_API int sb_alloc(size_t bytes, void **out_dev);
SB_API int sb_free(void *dev);
SB_API int sb_memset(void *dev, int value, size_t bytes, void *stream);
SB_API int sb_upload(void *dst_dev, const void *src_host, size_t bytes, void *stream);
SB_API int sb_download(void *dst_host, const void *src_dev, size_t bytes, void *stream);
SB_API int sb_host_alloc(size_t bytes, void **out_host); /* pinned */
SB_API int sb_host_free(void *host);

SB_API int sb_stream_create(void **out_stream);
SB_API int sb_stream_destroy(void *stream);
SB_API int sb_stream_sync(void *stream);
SB_API int sb_event_create(void **out_event);
SB_API int sb_event_destroy(void *event);
SB_API int sb_event_record(void *event, void *stream);
SB_API int sb_event_sync(void *event);
SB_API int sb_event_elapsed_ms(void *start, void *stop, float *out_ms);

/* CUDA-graph capture of a sequence of launches on `stream` (replaces CommandGraph). */
SB_API int sb_graph_begin(void *stream);
SB_API int sb_graph_end(void *stream, void **out_graph);
SB_API int sb_graph_launch(void *graph, void *stream);
SB_API int sb_graph_destroy(void *graph);

/* ---- weights ---- */

/* Bytes of one row of `k` weights in `format` as a GGUF stores it; 0 if k is not whole blocks. */
SB_API uint64_t sb_row_bytes(uint32_t format, uint32_t k);

/* fp32 (out_f16 == 0) or fp16-rounded-once (out_f16 != 0) values of `rows` native rows: the
 * device twin of the reference's dequantization check (dev/tests/engine/gguf_dequant_test.mm:50-56,
 * runtime/metal/kernels/common/gguf_staged.h:11-17). */
SB_API int sb_dequant(void *stream, uint32_t format, const void *weights_dev, uint32_t rows, uint32_t k, void *out_dev,
                      uint32_t out_f16);

/* ---- quantized linear: Y[M,N] = X[M,K] W[N,K]^T ----
 * Replaces ops::Linear::add -> addGgufStaged / addGgufColumn (runtime/ops/LinearGguf.cpp:212-362) and
 * the kernels gguf_decode_<fmt>_m*_{a,a_f32,r,g}, gguf_decode_*_gate_up
 * (runtime/metal/kernels/shared/gguf_linear.metal:113-130). */
typedef struct SbLinearArgs {
  const void *weights;  /* [n] native rows of k weights (gate rows for SB_EPILOGUE_GATE_UP) */
  const void *weights2; /* SB_EPILOGUE_GATE_UP: the up tensor's [n] rows; else NULL */
  const void *x;        /* bf16 [rows, x_stride]; may be NULL when `prepared` is given */
  const void *prepared; /* optional: the input already converted by sb_linear_prepare for this format's
                           layout (one conversion can feed several projections of the same input) */
  const void *aux;      /* bf16 [rows, aux_stride]: residual or gate, by epilogue; else NULL */
  void *out;            /* bf16 or fp32 [rows, out_stride] */
  const void *norm_weight; /* optional fused RMSNorm of x before the product: fp32 [k] weights, or NULL.
                              y = bf16((x * rsqrt(mean x^2 + 1e-6)) * w), then the product
                              (runtime/metal/kernels/shared/normalization.metal:60-94). */
  uint32_t format;      /* SB_FMT_Q4K / Q6K / Q80 */
  uint32_t n, k;        /* output columns (per tensor), input size */
  uint32_t rows;        /* M, the step's rows */
  uint32_t x_stride, aux_stride, out_stride; /* in elements */
  uint32_t epilogue;    /* SB_EPILOGUE_* */
  uint32_t out_f32;     /* 1: fp32 destination (logits) */
  uint32_t flags;       /* SB_LINEAR_* */
} SbLinearArgs;

enum {
  SB_LINEAR_PDL = 1 /* launch with programmatic stream serialization: the weight stream starts while the
                       producer of x drains */
};

/* Converts a projection input once into the fragment-ordered fp16 form the product reads
 * (the reference's prepared input: ops::LinearBuffers::prepared / PreparedInput,
 * runtime/ops/Linear.hpp:265-347; kernel decode_linear_gguf_prepare). `format` selects the layout
 * (Q4_K's differs from Q6_K / Q8_0's). An RMSNorm is fused in front when norm_weight is given. */
SB_API uint64_t sb_linear_prepared_bytes(uint32_t k);
SB_API int sb_linear_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride,
                             const void *norm_weight, uint32_t format, void *prepared_out, uint32_t flags);

/* Scratch (split-K partials and arrival counters) the context keeps for sb_linear; sized by
 * sb_init for the largest projection of the supported shapes and reused serially within a stream,
 * counters left at zero by the kernel that used them (runtime/ops/Linear.hpp:169-182). */
SB_API int sb_linear(void *stream, const SbLinearArgs *args);

/* The plan sb_linear will use for a shape: k-slices, CTAs, tile rows, ring stages, shared bytes.
 * (runtime/ops/Linear.hpp:287-301 `plan` is a value object shared by sizing and encoding.) */
typedef struct SbLinearPlan {
  uint32_t slices, ctas, tile_rows, stages, smem_bytes, stage_blocks, slice_blocks_max, tiles;
} SbLinearPlan;
SB_API int sb_linear_plan(uint32_t format, uint32_t n, uint32_t k, uint32_t rows, uint32_t epilogue,
                          SbLinearPlan *out_plan);

#ifdef __cplusplus
}
#endif
#endif /* SPLASH_B200_H */
