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
  SB_EPILOGUE_GATE_UP = 3,      /* one pass over gate and up rows: bf16(bf16(up) * silu(bf16(gate))) */
  SB_EPILOGUE_PARTIALS = 4,     /* no reduction: out is fp32 [slices of sb_linear_plan][16][out_stride] and receives every
                                   k-slice's sums; sb_linear_prepare_sum adds them (and a residual) where the sum is
                                   consumed, which takes the split-K exchange off the projection's tail */
  SB_EPILOGUE_GATE_UP_PARTIALS = 5 /* SB_EPILOGUE_GATE_UP without the reduction: out is fp32 [slices][16][out_stride] with
                                   the gate sums of column c at c and the up sums at n + c (out_stride >= 2 n);
                                   sb_linear_prepare_gate_up adds the slices and applies the activation where the
                                   result is consumed (same bits; measured no faster than the one-pass epilogue on the
                                   27B shape, whose two slices exchange cheaply, so the model driver does not use it) */
};

/* ---- context, memory, streams, events (replaces MetalBackend's buffer and command API) ---- */

SB_API int sb_device_count(void);
SB_API int sb_init(int device);
SB_API const char *sb_last_error(void);
/* Reads and clears the device status word (0 = healthy). Synchronizes the device. */
SB_API int sb_device_status(uint32_t *status);
SB_API int sb_sm_count(void);
/* Programmatic dependent launch (kernel prologues overlap the previous kernel's tail) for the small
 * kernels of this context; on by default. sb_linear takes it per call (SB_LINEAR_PDL). */
SB_API int sb_set_pdl(int enabled);
/* Which sb_attn_verify kernel runs: SB_ATTENTION_TCGEN05 (default; S and O in tensor memory) or
 * SB_ATTENTION_WARP_MMA (mma.sync; also taken when rows x group exceeds 128). Same results contract. */
enum { SB_ATTENTION_TCGEN05 = 0, SB_ATTENTION_WARP_MMA = 1 };
SB_API int sb_set_attention_kernel(int kind);

/* Device buffers. An allocation is held by whoever allocated it and by every live view of it; sb_free lets one holder
 * go (an allocation's own, given its base address; a view's, given the view's address) and the memory returns to the
 * driver with the last one, so a view keeps its base alive (the reference's ref-counted buffer handles,
 * runtime/metal/MetalBackend.hpp:42-78). sb_view checks [offset, offset + bytes) against the allocation that holds
 * base_dev (itself a base or a view) and fails with SB_ERR_INVALID when it runs past it. */
SB_API int sb_alloc(size_t bytes, void **out_dev);
SB_API int sb_view(void *base_dev, size_t offset, size_t bytes, void **out_view);
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
/* Completion without blocking (*out_done 1 or 0), and a wait that gives up: SB_ERR_BUSY after timeout_ms with the event
 * still pending (the reference's bounded wait on a ticket, runtime/metal/MetalBackend.hpp:468-478). */
SB_API int sb_event_query(void *event, int *out_done);
SB_API int sb_event_wait_bounded(void *event, uint32_t timeout_ms);
SB_API int sb_event_elapsed_ms(void *start, void *stop, float *out_ms);

/* CUDA-graph capture of a sequence of launches on `stream` (replaces CommandGraph). */
SB_API int sb_graph_begin(void *stream);
SB_API int sb_graph_end(void *stream, void **out_graph);
SB_API int sb_graph_launch(void *graph, void *stream);
SB_API int sb_graph_destroy(void *graph);
/* The reference's submission rule on top of sb_graph_launch: exactly one command in flight
 * (runtime/metal/MetalBackend.hpp:371-375). sb_submit launches the graph and hands out a ticket; a second sb_submit
 * before that ticket is consumed fails with SB_ERR_BUSY and enqueues nothing. sb_ticket_wait consumes the ticket once the
 * command has completed, or returns SB_ERR_BUSY after timeout_ms and leaves the ticket out. sb_graph_launch itself
 * stays unguarded for callers that order their work by streams and events. */
SB_API int sb_submit(void *graph, void *stream, uint64_t *out_ticket);
SB_API int sb_ticket_wait(uint64_t ticket, uint32_t timeout_ms);

/* Bytes of an argument structure of this header by its name ("SbLinearArgs", "SbGdnArgs", ...), 0 for an unknown name: lets a
 * binding in another language check its mirror of the structure against the library it loaded. */
SB_API uint64_t sb_struct_bytes(const char *name);

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
  SB_LINEAR_PDL = 1, /* launch with programmatic stream serialization: the weight stream starts while the
                        producer of x drains */
  SB_LINEAR_WIDE_IMAGE = 4, /* sb_linear_wide: weights / weights2 point to images made by sb_linear_wide_image (Q6_K, Q8_0, NVFP4) */
  SB_LINEAR_TCGEN05 = 2 /* Q4_K only: multiply on the tcgen05 tensor cores (weights expanded straight into tensor
                           memory, 128-row tiles) instead of warp-level MMA. Give the same flag to
                           sb_linear_prepare: the kernel reads its activations in another tile order. Same
                           results contract; at 16 rows the warp-level kernel is the faster one on B200. */
};

/* Converts a projection input once into the fragment-ordered fp16 form the product reads
 * (the reference's prepared input: ops::LinearBuffers::prepared / PreparedInput,
 * runtime/ops/Linear.hpp:265-347; kernel decode_linear_gguf_prepare). `format` selects the layout
 * (Q4_K's differs from Q6_K / Q8_0's). An RMSNorm is fused in front when norm_weight is given; normed_out
 * (optional, bf16 [rows, k]) also receives the normalised rows for the fp32 side projections. */
SB_API uint64_t sb_linear_prepared_bytes(uint32_t k);
SB_API int sb_linear_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride,
                             const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out, uint32_t flags);
/* The same over x = bf16(residual + sum of `slices` partial sums (fp32 [slices][16][partial_stride], as
 * SB_EPILOGUE_PARTIALS writes them, added in slice order)): the residual epilogue of the projection that produced the
 * partials, moved in front of the next projection's input conversion. sum_out (bf16 [rows, sum_stride]) receives x,
 * the new hidden state. */
SB_API int sb_linear_prepare_sum(void *stream, const float *partials, uint32_t slices, uint32_t partial_stride, const void *residual,
                                 uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                                 const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out, uint32_t flags);

/* The conversion for the projection that follows a gate/up pair left as SB_EPILOGUE_GATE_UP_PARTIALS: x = bf16(bf16(up) *
 * silu(bf16(gate))) with gate and up the slices' sums in slice order, i.e. the one-pass SwiGLU epilogue
 * (runtime/metal/kernels/shared/gguf_linear.metal:38) done where its result is read. n = the intermediate width (the
 * conversion's k); act_out (bf16 [rows, act_stride]) receives x. */
SB_API int sb_linear_prepare_gate_up(void *stream, const float *partials, uint32_t slices, uint32_t partial_stride, uint32_t n,
                                     void *act_out, uint32_t act_stride, uint32_t rows, uint32_t format, void *prepared_out,
                                     uint32_t flags);

/* Scratch (split-K partials and arrival counters) the context keeps for sb_linear; sized by
 * sb_init for the largest projection of the supported shapes and reused serially within a stream,
 * counters left at zero by the kernel that used them (runtime/ops/Linear.hpp:169-182). */
SB_API int sb_linear(void *stream, const SbLinearArgs *args);

/* ---- many rows (17 and up): the same product on the tcgen05 tensor cores with the weights dequantized to half ----
 * Replaces the reference's many-row projection tile (gguf_prefill_<fmt>_{a,r,g}, runtime/metal/kernels/shared/gguf_linear.metal,
 * geometry runtime/metal/abi/Gguf.h:31-35; the 64-row decode tiles of runtime/ops/Linear.hpp:94-97) and follows its
 * arithmetic: weights rounded to half once dequantized (runtime/metal/kernels/common/gguf_staged.h:11-57), fp32 sums, one
 * rounding after the epilogue. Q4_K; epilogues none / residual / up-with-gate / one-pass gate-up. Rows beyond 128 run as
 * passes of 128 over the weights. sb_linear forwards calls with more than 16 rows here. `prepared`, if given, is the
 * output of sb_linear_wide_prepare for the same rows and k (another layout than sb_linear_prepare's). */
SB_API uint64_t sb_linear_wide_prepared_bytes(uint32_t rows, uint32_t k);
SB_API int sb_linear_wide_prepare(void *stream, const void *x, uint32_t rows, uint32_t k, uint32_t x_stride, const void *norm_weight,
                                  void *prepared_out, uint32_t flags);
/* Q6_K, Q8_0 and NVFP4 rows are not 16-byte multiples (and Q6_K's codes are spread over bit planes), so the many-row kernel reads an
 * image of them, made once when the weights are loaded (as the reference prepares its GGUF tensors when it loads them,
 * runtime/model/GgufPreparation.hpp): per super-block the same codes re-ordered for the expansion and the block's scales
 * already multiplied out and rounded to half with a power of two per row taken out (Q6_K 224 bytes: d * sc; NVFP4 160
 * bytes: e4m3 * g; Q8_0 272 bytes: eight blocks' codes + 128 and their d), then one fp32 power of two per row. The weight's half is fl16(code * fl16(scale)): two roundings.
 * sb_linear_wide takes the image as `weights` with SB_LINEAR_WIDE_IMAGE. */
SB_API uint64_t sb_linear_wide_image_bytes(uint32_t format, uint32_t n, uint32_t k);
SB_API int sb_linear_wide_image(void *stream, uint32_t format, const void *weights, uint32_t n, uint32_t k, void *image_out);
/* Split K for narrow projections (n below what fills the SMs): with SB_EPILOGUE_PARTIALS the launch divides k into
 * sb_linear_wide_splits(n, k) ranges and out receives every range's sums, fp32 [splits][rows][out_stride];
 * sb_linear_wide_prepare_sum is then the next projection's conversion over x = bf16(residual + the splits' sums in split
 * order), x also written to sum_out (bf16 [rows, sum_stride]): the residual epilogue moved in front of its consumer, as
 * sb_linear_prepare_sum does for 16 rows. */
SB_API uint32_t sb_linear_wide_splits(uint32_t n, uint32_t k);
SB_API int sb_linear_wide_prepare_sum(void *stream, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual,
                                      uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                                      const void *norm_weight, void *prepared_out, uint32_t flags);
/* Either of the two conversions above (partials NULL: sb_linear_wide_prepare of x_or_sum_out; else sb_linear_wide_prepare_sum
 * into it) that also stores the normalised rows, bf16 [rows][k], as the fp32 side projections of the same input read them
 * (the GDN alpha / beta rows, the MoE router): what a separate sb_rmsnorm over the same rows would give, from the
 * conversion's own row statistics. Needs norm_weight. */
SB_API int sb_linear_wide_prepare_normed(void *stream, const float *partials, uint32_t splits, uint32_t partial_stride, const void *residual,
                                         uint32_t residual_stride, void *x_or_sum_out, uint32_t x_stride, uint32_t rows, uint32_t k,
                                         const void *norm_weight, void *prepared_out, void *normed_out, uint32_t flags);
SB_API int sb_linear_wide(void *stream, const SbLinearArgs *args);

/* The plan sb_linear will use for a shape: k-slices, CTAs, tile rows, ring stages, shared bytes.
 * (runtime/ops/Linear.hpp:287-301 `plan` is a value object shared by sizing and encoding.) */
typedef struct SbLinearPlan {
  uint32_t slices, ctas, tile_rows, stages, smem_bytes, stage_blocks, slice_blocks_max, tiles;
} SbLinearPlan;
SB_API int sb_linear_plan(uint32_t format, uint32_t n, uint32_t k, uint32_t rows, uint32_t epilogue,
                          SbLinearPlan *out_plan);
/* The same for a call that carries `flags` (SB_LINEAR_TCGEN05 selects the 128-row tensor-memory kernel's plan). */
SB_API int sb_linear_plan_flags(uint32_t format, uint32_t n, uint32_t k, uint32_t rows, uint32_t epilogue, uint32_t flags,
                                SbLinearPlan *out_plan);


/* ---- glue operators ---- */

/* y = bf16((x * rsqrt(mean x^2 + 1e-6)) * w), w fp32 [width]. Replaces ops::Normalization::addRms
 * (runtime/ops/Normalization.cpp:17-42; kernel norm_rms_row, runtime/metal/kernels/shared/normalization.metal:60-94). */
SB_API int sb_rmsnorm(void *stream, const void *x, uint32_t rows, uint32_t width, uint32_t x_stride, const void *weight,
                      void *out, uint32_t out_stride);

/* Token row gather with dequantization to bf16; a token outside the table reads row 0. Replaces
 * ops::Embedding::add (runtime/ops/Embedding.hpp:13-17; runtime/metal/kernels/shared/embedding.metal:10-18). */
SB_API int sb_embed(void *stream, uint32_t format, const void *table, uint32_t vocab, uint32_t width,
                    const uint32_t *tokens_dev, uint32_t rows, void *out, uint32_t out_stride);

/* cos/sin [rows][pairs] at positions[row] (device u32), angle = float(position) * inv_freq[pair].
 * Replaces ops::RoPE::addTreeTables (runtime/ops/RoPE.hpp:12-45; runtime/metal/kernels/shared/rope.metal:50-76):
 * the caller writes position = anchor + tree depth per row. */
SB_API int sb_rope_tables(void *stream, const uint32_t *positions_dev, uint32_t rows, const float *inv_freq_dev,
                          uint32_t pairs, float scale, float *cos_dev, float *sin_dev);

/* fp32 projection of plain fp32 rows: out[rows, n] = x[rows, k] w[n, k]^T, bf16 or fp32 out.
 * Replaces ops::addGgufFloat (runtime/ops/LinearGguf.cpp:559-604; runtime/metal/kernels/shared/gguf_float.metal:1-8):
 * the GDN alpha/beta rows and the MoE router. */
SB_API int sb_linear_f32(void *stream, const float *w_dev, const void *x, uint32_t rows, uint32_t n, uint32_t k,
                         uint32_t x_stride, void *out, uint32_t out_stride, uint32_t out_f32, const void *norm_weight);

/* ---- steps of several lanes ----
 * A step may carry several lanes (concurrent requests), each with its own block of rows (the reference's StepRows /
 * SplashLaneRows, runtime/ops/LaneRows.hpp:36-62, runtime/metal/abi/VerifyTree.h:38-45). Here a lane has 16 row slots: lane l's
 * rows are rows 16 l .. 16 l + rows - 1 of every row-indexed buffer (packed rows, queries, tokens, tree rows, logits, outputs),
 * its uniforms the 80 from 80 l on, its results the 4 words from 4 l on, and every per-lane state buffer (positions, page
 * tables, GDN cells and tapes, penalty tables) is an array over the lanes of the one-lane buffer. The operators below take
 * `lanes` (0 or 1: one lane, the layout above with l = 0) and spread the lanes over their grids; `rows` stays the rows of
 * one lane. The projections see the step's rows as one matrix of 16 x lanes rows (sb_linear / sb_linear_wide). */

/* ---- INT8 paged KV attention ---- */

/* One attention layer's cache: pages of page_tokens tokens; keys and values token-major
 * [page][kv_head][token][dim] int8; one scale per (token, kv head), fp32 (scale_f16 = 0, the
 * reference's: runtime/ops/PagedKv.hpp:223-232) or fp16. */
typedef struct SbKvLayer {
  void *k, *v, *k_scale, *v_scale;
  uint32_t kv_heads, head_dim, page_tokens, scale_f16;
} SbKvLayer;

/* Per row: per-head RMSNorm of q and k, partial RoPE of pairs (i, i + pairs), queries staged
 * [row][q_head][dim] bf16, K and V rows quantized into the slot of token committed + row:
 * scale = max|x| / 127, code = clamp(rint(x * 127 / max), -127, 127). Replaces
 * ops::PagedAttention::addProjection (runtime/metal/kernels/common/attention_qkv_prepare.h:26-91,
 * attention_store.h:52-85). qkv row = [q_heads x (q[D], gate[D] if gated)][kv_heads x k][kv_heads x v]. */
typedef struct SbAttnStoreArgs {
  const void *qkv;          /* bf16 [rows, qkv_stride] */
  const float *q_norm, *k_norm; /* fp32 [head_dim] */
  const float *cos_tab, *sin_tab; /* fp32 [rows, pairs] */
  const uint32_t *page_table; /* device u32 physical page per logical page */
  void *queries;            /* bf16 [rows, q_heads, head_dim] */
  SbKvLayer cache;
  const uint32_t *committed_dev; /* optional device word overriding `committed`, so a captured graph follows the lane;
                                    with lanes: one word per lane (required) */
  uint32_t rows, q_heads, gated, pairs, qkv_stride, committed;
  uint32_t lanes;             /* 0 or 1: one lane */
  uint32_t page_table_stride; /* entries between consecutive lanes' page tables */
} SbAttnStoreArgs;
SB_API int sb_attn_store(void *stream, const SbAttnStoreArgs *args);

/* Attention of the step's rows over the stored pages, one launch: a split-KV page loop per (kv head,
 * split) with online softmax, the splits merged in split order, output gated by sigmoid(gate) where
 * gated. Row r sees tokens [0, committed + r]; with `tree` (SplashTreeRow: ancestors u32, parent u16,
 * depth u16; runtime/metal/abi/VerifyTree.h:24-28) block rows are limited to the row's ancestors.
 * Replaces ops::PagedAttention::addAttention (runtime/metal/kernels/common/paged_attention_tile.h:339-535,
 * attention_gate.h:19-45). */
typedef struct SbAttnArgs {
  const void *queries;      /* bf16 [rows, q_heads, head_dim] from sb_attn_store */
  const void *qkv;          /* the packed rows, for the gates (NULL when not gated) */
  const uint32_t *page_table;
  const void *tree;         /* optional device SplashTreeRow[rows] */
  void *out;                /* bf16 [rows, out_stride] = [row][q_head][dim] */
  SbKvLayer cache;
  const uint32_t *committed_dev; /* optional device word; `committed` is then the bound the split plan is made for; with lanes:
                                    one word per lane (required), `committed` the largest */
  uint32_t rows, q_heads, gated, qkv_stride, out_stride, committed;
  uint32_t lanes;             /* 0 or 1: one lane; else the lanes share the launch (fewer splits a lane) */
  uint32_t page_table_stride; /* entries between consecutive lanes' page tables */
} SbAttnArgs;
SB_API int sb_attn_verify(void *stream, const SbAttnArgs *args);

/* Moves the accepted path's rows (codes and scales) from slot committed + row to slot
 * committed + depth, in depth order; nothing moves for a chain. Replaces
 * ops::PagedAttention::addPathCommit (runtime/metal/kernels/shared/kv_path_commit.metal:21-46).
 * path_mask_dev: device u32, the accepted path's row mask (sb_accept's retained_rows). */
SB_API int sb_kv_path_commit(void *stream, const SbKvLayer *cache, const uint32_t *page_table, uint32_t committed,
                             const uint32_t *path_mask_dev);
/* The same for the lanes of a step: lane l's position committed_dev[l], its page table page_table_stride entries after lane
 * l - 1's, its path mask mask_stride words after lane l - 1's (4 for the results of sb_accept). */
SB_API int sb_kv_path_commit_lanes(void *stream, const SbKvLayer *cache, const uint32_t *page_table, uint32_t page_table_stride,
                                   const uint32_t *committed_dev, const uint32_t *path_mask_dev, uint32_t mask_stride, uint32_t lanes);
/* The same with the lane's position read from a device word, so a captured graph follows the lane. */
SB_API int sb_kv_path_commit_at(void *stream, const SbKvLayer *cache, const uint32_t *page_table, const uint32_t *committed_dev,
                                const uint32_t *path_mask_dev);

/* ---- Gated DeltaNet verify step ---- */

typedef struct SbGdnTape {
  void *inputs; /* bf16 [rows, conv_dim] conv inputs */
  void *k;      /* bf16 [rows, key_heads * 128] */
  void *v;      /* bf16 [rows, value_heads * 128] */
  void *beta;   /* bf16 [rows, value_heads] */
  float *decay; /* fp32 [rows, value_heads] */
} SbGdnTape;

/* One lane, one layer: fold the first pending_rows rows of the previous step's tape into the state
 * (stored as the committed state), then conv + SiLU, q/k norm, gates, the chain scan from the committed
 * state (outputs only), gated RMSNorm, and this step's tape. pending_rows_dev (optional device u32)
 * overrides pending_rows so acceptance can stay on the device. Replaces ops::GDN::addDecode / addFold
 * (runtime/ops/GDN.cpp:225-328; runtime/metal/kernels/decode/gdn.metal:139-616). State fp32
 * [value_head][value dim 128][key dim 128]. */
typedef struct SbGdnArgs {
  const void *qkvz;        /* bf16 [rows, qkvz_stride]: q | k | v | z */
  const void *b, *a;       /* bf16 [rows, ab_stride]; unused (may be null) with gate_weight */
  const void *conv_w;      /* bf16 [conv_dim, 4] */
  const float *a_scale;    /* fp32 [value_heads] */
  const void *dt_bias;     /* bf16 [value_heads] */
  const float *norm_w;     /* fp32 [128] */
  const void *conv_state_in; /* bf16 [3, conv_dim] */
  void *conv_state_out;
  const float *state_in;
  float *state_out;
  SbGdnTape pending, step;
  void *hidden;            /* bf16 [rows, hidden_stride] */
  const uint32_t *pending_rows_dev;
  uint32_t rows, pending_rows, key_heads, value_heads, qkvz_stride, ab_stride, hidden_stride, tiled;
  /* Optional fused gate projection (ops::addGgufFloat of the alpha / beta rows, runtime/ops/LinearGguf.cpp:559-604,
   * inside the same kernel): when gate_weight is given, b and a are not read; row r's b for head h is
   * bf16(gate_input[r] . gate_weight[h]) and its a is bf16(gate_input[r] . gate_weight[value_heads + h]), summed in
   * sb_linear_f32's order, so both ways give the same bits. */
  const float *gate_weight; /* fp32 [2 * value_heads, gate_k]: the b rows, then the a rows */
  const void *gate_input;   /* bf16 [rows, gate_input_stride]: the normalised layer input */
  uint32_t gate_k, gate_input_stride;
  /* Trees (runtime/metal/kernels/decode/gdn.metal:131-137, 198-207, 418-478). tree: device SplashTreeRow[rows] (NULL: the
   * rows are a chain); a row's convolution taps its path's last tokens and its output is the state after its own path:
   * S_committed z + sum_j c_j v_j with the query transformed up the path, z_j-1 = d_j (z_j - c_j k_j),
   * c_j = beta_j (k_j . z_j). pending_path: the row mask, in the pending tape, of the path the previous step accepted
   * (sb_accept's retained_rows), folded in depth order; pending_path_dev the same as a device word; neither given, the
   * pending tape's first pending_rows rows. */
  const void *tree;
  const uint32_t *pending_path_dev;
  uint32_t pending_path;
  uint32_t flags;           /* SB_GDN_* */
  uint32_t lanes;           /* 0 or 1: one lane. Else state_in / state_out, the carried convolution rows and both tapes are arrays
                               over the lanes, pending_rows_dev / pending_path_dev one word per lane (the host values
                               pending_rows / pending_path then apply to every lane), the rows of lane l at 16 l */
  uint32_t reserved;
} SbGdnArgs;
enum {
  SB_GDN_STATE_SETTLED = 1 /* the caller vouches that no launch still running on the stream writes state_in, so the kernel
                              may fetch the cell before it waits for the launch ahead (the model's step: the cell was written
                              a whole step earlier). Without the flag every read waits, which is what a fold followed at
                              once by a step on the swapped cells needs (ops::GDN::addFold then addDecode). */
};
SB_API int sb_gdn_verify(void *stream, const SbGdnArgs *args);

/* sb_gdn_verify for callers that cannot allocate device memory: a process whose GPU memory is already handed out
 * in full to its own arena, a plugin inside one, code running under a fixed memory budget. It has no counterpart
 * in the reference. Same arguments and results as sb_gdn_verify; it needs no sb_init and calls no cudaMalloc,
 * cudaFree or any other allocating routine. Its scratch (the recurrent rows awaiting their gate and one arrival
 * counter per value head, 256 KiB + 256 bytes) is an array built into the library, so every GPU that loads the
 * library holds it until the process exits, and the shape is limited to 64 value heads (more fails with
 * SB_ERR_INVALID).
 * The first call on each device looks up the array's device address (with that device current); make that first
 * call outside any stream capture. All calls share the one array: it keeps the previous call's contents (this
 * call clears the counters it needs at zero on `stream`), and two calls that overlap on the GPU - different
 * streams, or concurrent processes' threads on one context - race on it. */
SB_API int sb_gdn_verify_static(void *stream, const SbGdnArgs *args);

/* ---- selection and acceptance ---- */

/* Selection of every row of one lane's chain. temperature 0: greedy (largest finite logit, ties to the
 * lowest id, none -> 0xFFFFFFFF). Else weights exp((l - max) / T) of the tokens before the distribution's end (min_p,
 * top_k, top_p below), shards of 256 ids summed in id order and
 * the shards in order; the drafted child (input token of row r + 1) is kept iff u_child * Z < w_child, else
 * the row draws from the residual with its own uniform; the last row draws from the full distribution.
 * uniforms (device fp32): [0,16) row draws, 16 + 4 * row child tests (runtime/metal/abi/Sampling.h:12-31).
 * Replaces ops::Sampling::addVerify (runtime/ops/Sampling.cpp:198-328; runtime/metal/kernels/decode/sampling.metal
 * :1896-1991 greedy, :713-885 draw). */
typedef struct SbLanePolicy {
  float temperature; /* 0: greedy */
  float min_p;       /* 0: off */
  uint32_t top_k;    /* 0: off */
  float top_p;       /* 1: off */
} SbLanePolicy;
typedef struct SbSampleArgs {
  const float *logits;       /* fp32 [rows, logit_stride] */
  const uint32_t *input_tokens; /* device u32 [rows] */
  const float *uniforms;     /* device fp32 [80], or NULL for greedy */
  uint32_t *selected;        /* device u32 [rows] */
  float *workspace;          /* device fp32, rows * (2 * shards + 8) */
  uint32_t rows, vocab, logit_stride;
  float temperature;
  /* The end of the distribution a sampled row draws from (runtime/metal/kernels/decode/sampling.metal:604-668), in the
   * order logit descending, id ascending: tokens weighing at least min_p of the heaviest (0: off), then the top_k
   * first of those (0 or >= vocab: off), then the shortest prefix whose mass exceeds top_p of what those two keep
   * (0 or >= 1: off; ties at the last logit keep their lowest ids). Vocabulary up to 262144 when any is on. */
  float min_p;
  uint32_t top_k;
  float top_p;
  uint32_t *cut_out;         /* optional device u32 [rows, 2]: the end as {order key of the last logit, last id} */
  /* Optional: the children each row's draft drew, for recursive rejection sampling without replacement
   * (runtime/metal/kernels/decode/sampling.metal:693-885; uniforms runtime/metal/abi/Sampling.h:12-31). Per row its 16
   * draft candidates (token ids, 0xFFFFFFFF past the draft's list), the draft's probabilities q of them, and the candidate
   * indices of up to 4 drawn children in the order drawn (0xff past them). Child c of row r is kept iff
   * u[16 + 4 r + c] q < p (p its probability under the target); after a rejection the target becomes max(p - q, 0)
   * renormalised and the draft loses the child; a row that keeps none draws with u[r] from the last residual, its
   * candidates first, then the tokens outside them by the target's own weights. Without these the drafted child is the
   * input token of row r + 1 with q = 1 (a chain from a deterministic draft), which is the same rule. */
  const uint32_t *candidate_ids; /* device u32 [rows, 16] or NULL */
  const float *candidate_q;      /* device fp32 [rows, 16] */
  const uint8_t *draws;          /* device u8 [rows, 4] */
  uint32_t lanes;                /* 0 or 1: one lane */
  uint32_t reserved;
  /* Optional: a policy a lane (device SbLanePolicy [lanes]), read by the kernel in place of temperature / min_p / top_k /
   * top_p above, so the lanes of one step may be greedy and sampled side by side (the reference's policies a lane,
   * Sampling::addVerify's `policies`, runtime/ops/Sampling.hpp:58-85) and may change between replays of a captured step.
   * Needs uniforms and the workspace. */
  const struct SbLanePolicy *lane_policies;
} SbSampleArgs;
/* The sampling penalties of one lane's rows, in place, before selection: a token the prompt or the output holds has a
 * positive logit divided and a negative one multiplied by `repetition`; a token the output holds `count` times is
 * lowered by frequency * count + presence; the result saturates at the largest finite value; NaN and -inf stay.
 * words (device u32 [vocab]): the output's count of each token in the low 31 bits, bit 31 set when the prompt holds
 * it; a row's context also counts the draft tokens (input rows 1..) on its path in `tree`, but the anchor. Replaces
 * ops::Sampling's penalty pass (kernel decode_sample_penalize, runtime/metal/kernels/decode/sampling.metal:985-1048;
 * SamplingPenaltyParams, runtime/metal/abi/Sampling.h:124-145). */
typedef struct SbPenaltyArgs {
  float *logits;                /* device fp32 [rows, logit_stride] */
  const uint32_t *words;        /* device u32 [vocab] */
  const uint32_t *input_tokens; /* device u32 [rows] */
  const void *tree;             /* device SplashTreeRow[rows] */
  uint32_t rows, vocab, logit_stride;
  float repetition, presence, frequency;
  uint32_t lanes;               /* 0 or 1: one lane; else `words` is [lanes][vocab] */
  uint32_t reserved;
} SbPenaltyArgs;
SB_API int sb_sample_penalize(void *stream, const SbPenaltyArgs *args);

/* The tokens a lane's rows may select, in place, before selection (the admission of the reference's selection kernels,
 * TargetRow::admits, runtime/metal/kernels/decode/sampling.metal:33-46; ops::SamplingBuffers::constraintMasks and
 * SamplingPolicy::constrained / excludesStopTokens, runtime/ops/Sampling.hpp:58-70,112): a token whose bit in the row's
 * constraint mask is clear, or that is one of `excluded` (the stop tokens of a lane that ignores end-of-sequence), gets the
 * logit -inf, which selection reads as not selectable; a row that admits nothing selects 0xFFFFFFFF. masks: device u32
 * [rows][mask_words], bit t % 32 of word t / 32 for token t, or NULL (unconstrained); excluded: device u32 [n_excluded]
 * (up to 16) or NULL. */
typedef struct SbAdmitArgs {
  float *logits;             /* device fp32 [rows, logit_stride] */
  const uint32_t *masks;     /* device u32 [rows, mask_words] or NULL */
  const uint32_t *excluded;  /* device u32 [n_excluded] or NULL */
  uint32_t rows, vocab, logit_stride, mask_words, n_excluded;
  uint32_t lanes;            /* 0 or 1: one lane; else rows 16 z .. of lane z */
} SbAdmitArgs;
SB_API int sb_sample_admit(void *stream, const SbAdmitArgs *args);

SB_API uint64_t sb_sample_workspace_bytes(uint32_t rows, uint32_t vocab);
SB_API int sb_sample_verify(void *stream, const SbSampleArgs *args);

/* Acceptance (runtime/metal/kernels/decode/sampling.metal:2044-2083; params AcceptBatchParams,
 * runtime/metal/abi/Sampling.h:314-317): follow from row 0 the child whose parent is the row and whose
 * input token equals the row's selection; kept = min(accepted + 1, remaining); the path's selections
 * move to the first kept slots of `tokens`; a stop token truncates. results (device u32[4]): retained,
 * accepted, retained_rows mask, 0. */
typedef struct SbAcceptArgs {
  const uint32_t *input_tokens; /* device u32 [rows] */
  const void *tree;             /* device SplashTreeRow[rows] */
  uint32_t *tokens;             /* device u32 [rows]: selections in, retained tokens out */
  uint32_t *results;            /* device u32 [4] */
  const uint32_t *stop_tokens;  /* device u32 [n_stop] or NULL */
  uint32_t rows, remaining, n_stop;
  uint32_t lanes;               /* 0 or 1: one lane; else results is [lanes][4] */
} SbAcceptArgs;
SB_API int sb_accept(void *stream, const SbAcceptArgs *args);

/* Selection and acceptance in one launch (the reference's verify selection ends in its acceptance the same way,
 * runtime/metal/kernels/decode/sampling.metal:1896-2083: the rows select, then the lane's path is walked): a block per
 * row selects as sb_sample_verify does; the block of a lane that finishes last walks the accepted path as sb_accept does
 * and, with `committed` given, commits the lane: advance 0 clears the lane's pending rows, 1 adds the retained rows to
 * committed[lane] and leaves them (and the path's row mask) pending for the next step's GDN fold, 2 leaves everything,
 * 3 | rows << 8 commits every row (SB_TARGET_PROMPT). accept.input_tokens = sample.input_tokens, accept.tokens =
 * sample.selected, same rows and lanes. tickets: device u32 [lanes], zero before the first call; the kernel returns
 * them to zero. Results equal those of the two separate calls bit for bit. */
typedef struct SbSelectAcceptArgs {
  SbSampleArgs sample;
  SbAcceptArgs accept;
  uint32_t *tickets;      /* device u32 [lanes] */
  uint32_t *committed;    /* device u32 [lanes] or NULL: no commit */
  uint32_t *pending_rows; /* device u32 [lanes] */
  uint32_t *pending_path; /* device u32 [lanes] */
  uint32_t advance, reserved;
  /* Optional: the rows each lane's block really holds (device u32 [lanes], each 0..sample.rows; the reference's SplashLaneRows,
   * runtime/ops/LaneRows.hpp:36-62): lanes step together with blocks of different lengths. A lane selects and accepts among
   * its own rows only (the slots past them hold whatever the caller left there and are never accepted), a prompt block
   * commits its own rows, and a lane of no rows keeps its position and gets results {0, 0, 0, 0}. NULL: sample.rows for all. */
  const uint32_t *lane_rows;
  /* Optional: how many more tokens each lane's request may take (device u32 [lanes], each at least 1; the `remaining` of the
   * reference's acceptance a lane, AcceptBatchParams, runtime/metal/abi/Sampling.h:314-317): a lane retains at most that
   * many tokens. NULL: accept.remaining for all. */
  const uint32_t *lane_remaining;
} SbSelectAcceptArgs;
SB_API int sb_select_accept(void *stream, const SbSelectAcceptArgs *args);

/* ---- the target model's verify step ----
 * The layer loop and the step's commit, as the reference's QwenTarget::addPrefillLayers /
 * encodeTargetDecodeForward / encodeVerifyCommit build them (runtime/model/QwenTarget.hpp:618-652,
 * runtime/model/QwenTarget.cpp:206-496, runtime/model/Runtime.cpp:2677-2717,2883-2892): pre-norm residual blocks,
 * layer l a full-attention layer iff (l + 1) % attention_interval == 0 (runtime/model/QwenHybridLayout.hpp:132-135),
 * else Gated DeltaNet; dense SwiGLU FFN; final norm and the vocabulary projection into fp32 logits of every row;
 * selection, acceptance, and the lane's commit (committed tokens and the GDN tape's accepted rows stay on the device).
 * One lane (batch 1) per target, or SbTargetConfig.lanes of them stepped together. */
typedef struct SbTargetConfig {
  uint32_t layers, hidden, vocab, intermediate;
  uint32_t q_heads, kv_heads, head_dim, rotary_pairs;
  float rope_theta;
  uint32_t gdn_key_heads, gdn_value_heads;
  uint32_t attention_interval;  /* 4 */
  uint32_t page_tokens, kv_scale_f16, max_context;
  uint32_t fmt_proj, fmt_down, fmt_head, fmt_embed; /* SB_FMT_* */
  uint32_t gated_attention, tiled_heads;
  /* Tensor parallelism: this process is rank tp_rank of tp_world ranks, one per GPU of the node (0 or 1: the whole
   * model on this GPU). The configuration above stays the whole model's; the rank holds its share (below). */
  uint32_t tp_world, tp_rank;
  /* MoE feed-forward blocks (runtime/model/Qwen3_6Moe.hpp:27-52) instead of dense ones when moe_experts > 0: a router over
   * moe_experts experts, the moe_top_k best per row, expert intermediate width moe_intermediate, and one shared expert
   * gated by a scalar per row; tensors ffn_router (fp32 [experts, hidden]), ffn_shared_gate (fp32 [hidden]),
   * ffn_gate_exps / ffn_up_exps ([experts + 1][moe_intermediate][hidden] rows of fmt_proj, the shared expert last),
   * ffn_down_exps ([experts + 1][hidden][moe_intermediate]). `intermediate` is then unused. Not with tensor parallelism. */
  uint32_t moe_experts, moe_top_k, moe_intermediate;
  /* Concurrent requests stepped together (0 or 1: one lane; up to 32): every per-lane buffer of the target becomes an array
   * over the lanes ("steps of several lanes" above), a layer's KV pool holds the lanes' pages one lane after the other, and
   * a step multiplies 16 x lanes rows on the many-row projection kernel, which needs Q4_K projections (fmt_proj, fmt_down,
   * fmt_head). One GPU (or expert-parallel ranks). */
  uint32_t lanes;
  /* Expert parallelism: this process is rank ep_rank of ep_world ranks (0 or 1: none), one per GPU of the node. Every rank
   * steps its own `lanes` lanes and holds the routed experts [ep_rank E / ep_world, ..) of every MoE block in its
   * ffn_*_exps tensors, then the shared expert ([E / ep_world + 1] experts); everything else whole. MoE models with
   * several lanes. The ranks' windows are connected with sb_target_tp_export / sb_target_tp_connect. */
  uint32_t ep_world, ep_rank;
} SbTargetConfig;

enum {
  SB_TARGET_ADVANCE = 1, /* the step commits: committed += retained, the next step folds the accepted rows */
  SB_TARGET_GRAPH = 2,   /* replay the step as a captured CUDA graph (captured on first use per parity) */
  SB_TARGET_TREE = 4,    /* the block is a tree: the target's `tree` buffer holds its SplashTreeRow rows (row 0 the anchor,
                            parents before children; runtime/metal/abi/VerifyTree.h:24-45) instead of the chain the step
                            writes there itself. Positions are the rows' depths, attention and GDN follow each row's path,
                            the accepted path's KV rows move to their depths, and the next step folds the path's tape
                            rows. The step after a tree step carries the flag too (a chain can be given as a tree). */
  SB_TARGET_KEEP_PENDING = 8, /* without SB_TARGET_ADVANCE: the lane's pending GDN rows (`pending_rows`, sb_target_tensor) stay
                            as they are instead of being cleared, so every such step folds the same rows again: a held
                            lane that still does a committing cycle's fold work (steady-state timing). */
  SB_TARGET_DRAWS = 16,  /* sampled rows (temperature > 0) take their children from the target's `candidates` (u32 [16][16]),
                            `candidate_q` (fp32 [16][16]) and `draws` (u8 [16][4]) buffers, which the host (the draft side)
                            fills before the step: recursive rejection sampling over up to 4 drawn children a row
                            (SbSampleArgs). A sampled tree block requires it; a sampled chain without it tests the next row's
                            input token with q = 1. */
  SB_TARGET_PROMPT = 32  /* with SB_TARGET_ADVANCE, chains only: the block's rows are tokens of the prompt (row 0 the first of them
                            that the target has not seen), and every row is committed whatever the target selected: results =
                            {rows, rows - 1, all rows}, the cache keeps the rows' K/V, the next step folds all of them into the
                            GDN state. `selected` row rows - 1 is the target's token after the block. A prompt enters the cache
                            this way, 16 tokens a step and lane, through the verify step's own kernels (the reference's prefill
                            path with its 128-row tiles, runtime/metal/kernels/prefill/, is a separate one). */
};

/* ---- MoE routing ----
 * Per row: the top_k experts by fp32 router score (descending score, then ascending id) and their weights: the softmax
 * of their scores, w_r = exp2((s_r - s_0) log2 e) / sum, or with sigmoid_normalized each one's sigmoid over the sum of
 * theirs; sums in rank order. With shared_gate (fp32 [input_size]) every row gets one more route, the shared expert
 * (id `experts`), weighted by sigmoid(input . shared_gate). Replaces MoE::addRouting's selection (kernel moe_route_select,
 * runtime/metal/kernels/shared/moe.metal:22-111); the scores come from sb_linear_f32 over the router's rows. */
typedef struct SbMoeRouteArgs {
  const float *scores;      /* device fp32 [rows, slots] */
  const void *input;        /* bf16 [rows, input_size]; with shared_gate */
  const float *shared_gate; /* fp32 [input_size] or NULL */
  uint32_t *selected;       /* device u32 [rows, top_k (+ 1)] */
  float *weights;           /* device fp32 [rows, top_k (+ 1)] */
  uint32_t rows, experts, slots, top_k, input_size, sigmoid_normalized;
} SbMoeRouteArgs;
SB_API int sb_moe_route(void *stream, const SbMoeRouteArgs *args);

/* The routed rows through their experts and back, for the rows of one lane's block (up to 16 rows x 32 routes):
 *   intermediate = bf16(bf16(up_e . x) * silu(bf16(gate_e . x))), y = bf16(down_e . intermediate) per route (row, expert e),
 *   out = bf16(residual + sum over the row's routes in slot order of weight * float(y)).
 * Replaces, in that regime, the expert passes and the combine of MoE::addRouted (runtime/ops/MoE.cpp:122-187,260-270;
 * runtime/metal/kernels/common/moe_gguf_expert_tile.h:33-84, runtime/metal/kernels/shared/moe_gguf.metal:94-160,
 * runtime/metal/kernels/shared/moe.metal:367-392). Every route streams its expert's rows by itself (a matrix-vector
 * product); the reference's grouping of routes into per-expert tiles, which pays from about 64 rows on, is not built.
 * gate, up: native Q4_K rows [experts_total][inter][hidden]; down: [experts_total][hidden][inter]; the shared expert,
 * if routed, is expert index `experts` of the same tensors (experts_total counts it). */
typedef struct SbMoeExpertArgs {
  const void *input;        /* bf16 [rows, hidden] */
  const void *residual;     /* bf16 [rows, hidden] or NULL */
  const uint32_t *selected; /* device u32 [rows, routes] from sb_moe_route */
  const float *weights;     /* device fp32 [rows, routes] */
  const void *gate, *up, *down;
  void *scratch;            /* sb_moe_scratch_bytes */
  void *out;                /* bf16 [rows, hidden] */
  uint32_t rows, routes, hidden, inter, format, experts_total;
} SbMoeExpertArgs;
SB_API uint64_t sb_moe_scratch_bytes(uint32_t rows, uint32_t routes, uint32_t hidden, uint32_t inter);
SB_API int sb_moe_experts(void *stream, const SbMoeExpertArgs *args);
/* A rank's share of an MoE block under expert parallelism: of the routes in `selected` (expert ids of the whole block) those
 * whose expert is one of [expert0, expert0 + experts_local), and those of the shared expert (id shared_id, if below
 * 0xffffffff) for rows [own_row0, own_row0 + own_rows). gate / up / down hold the rank's experts in order, then the shared
 * expert: experts_total = experts_local (+ 1). out: fp32 [rows, hidden], the weighted sums in slot order (no residual; rows
 * without a route here get zeros). Any number of rows (the grouped kernels); scratch as sb_moe_scratch_bytes with at
 * least 17 rows. */
SB_API int sb_moe_experts_partial(void *stream, const SbMoeExpertArgs *args, uint32_t expert0, uint32_t experts_local, uint32_t shared_id,
                                  uint32_t own_row0, uint32_t own_rows);

/* ---- tensor parallelism between the GPUs of one node ----
 * The reference runs on one GPU; its projections admit the usual split, and this is it: rank r of W holds
 *   q heads [r Q/W, (r+1) Q/W) with their KV heads (KV head r K/W when W > K: a KV head and its pages are then held
 *   by W/K ranks), GDN key and value heads [r K/W, ..) and [r V/W, ..) with their state, convolution channels and
 *   tapes, rows of in_proj / ssm_ab / ffn_gate / ffn_up for those heads and for its super-blocks of the intermediate
 *   width (68 super-blocks over 8 ranks: 9,9,9,9,8,8,8,8), the matching input columns of out_proj and ffn_down, and
 *   vocabulary columns in units of 64; norms and the embedding table whole.
 * out_proj and ffn_down then give each rank a share of the sum. The ranks exchange shares through each other's
 * memory (CUDA IPC mappings over NVLink, plain stores and loads: no TMA, no multicast) inside the kernel that
 * converts the next projection's input, and add them in rank order, so every rank holds the same hidden state bit
 * for bit; the logits' columns are gathered the same way and selection, acceptance and the commit run on every rank.
 * An exchange that waits longer than 2 s for a peer records a wait failure in the device status word
 * (sb_device_status) and carries on; later exchanges then do not wait.
 *
 * A group is one rank's end: create on every rank, pass every rank's exported handle to every rank (any host
 * transport), connect. `width` = the hidden size; `gather_width` = the vocabulary size. */
#define SB_TP_HANDLE_BYTES 64
SB_API int sb_tp_create(uint32_t world, uint32_t rank, uint32_t width, uint32_t gather_width, void **out_group);
SB_API int sb_tp_destroy(void *group);
SB_API int sb_tp_export(void *group, void *handle_out /* SB_TP_HANDLE_BYTES */);
SB_API int sb_tp_connect(void *group, const void *handles /* [world][SB_TP_HANDLE_BYTES], rank order */);
/* The group's fp32 [16][gather_width] matrix that sb_tp_all_gather completes on every rank. */
SB_API int sb_tp_gather_matrix(void *group, void **out_dev, uint64_t *out_bytes);
/* sb_linear_prepare_sum where the slices' sum is this rank's share of the whole: exchange, sum in rank order, residual,
 * conversion. `index` = the exchange's place among the step's exchanges (the same on every rank). k = the group's width. */
SB_API int sb_tp_prepare_sum(void *stream, void *group, uint32_t index, const float *partials, uint32_t slices, uint32_t partial_stride,
                             const void *residual, uint32_t residual_stride, void *sum_out, uint32_t sum_stride, uint32_t rows, uint32_t k,
                             const void *norm_weight, uint32_t format, void *prepared_out, void *normed_out, uint32_t flags);
/* This rank's columns [column0, column0 + columns) of the gather matrix go to every peer; returns (on the stream) when
 * every peer's columns have arrived here. */
SB_API int sb_tp_all_gather(void *stream, void *group, uint32_t index, uint32_t rows, uint32_t column0, uint32_t columns);
/* How the shares of a sum travel, for exchanges enqueued (or captured) after the call; the same on every rank. 1: every
 * rank sends its share to every rank and all add (one trip over NVLink, W - 1 copies); 2: shares go to the columns'
 * owner, which adds them and sends the finished bf16 values to every rank (two trips, 1 / W of the bytes); 0 (default):
 * one shot with two ranks, two shots with more. Either way every rank ends with the same bits. */
SB_API int sb_tp_set_exchange(int shots);
/* How long a kernel waits for another GPU's data (the tensor- and expert-parallel exchanges) before it records
 * SB_DEV_WAIT_EXPIRED in the device status word and carries on; 0 restores the default of 2 s. Kernels that find the status
 * word set do not wait at all, so a lost peer costs one limit, not one per exchange. */
SB_API int sb_set_wait_limit_ns(uint64_t ns);
/* Ends a step of `exchanges` exchanges: the next step's indices start over. (sb_target_* steps do this themselves.) */
SB_API int sb_tp_advance(void *stream, void *group, uint32_t exchanges);

/* ---- expert parallelism between the GPUs of one node ----
 * Rank r of W holds the routed experts [r E / W, (r + 1) E / W) of every MoE block (and a copy of the shared expert, which
 * it applies to its own rows) and steps its own lanes; the reference runs on one GPU (MoE::addRouted,
 * runtime/ops/MoE.cpp:122-187,260-270). A block's rows meet their experts in two exchanges through peer-mapped memory
 * (CUDA IPC windows over NVLink, plain stores and loads, bounded waits):
 *   sb_ep_dispatch  every rank's normalised rows (bf16 [rows, hidden]), routes and route weights ([rows, routes]) into
 *                   every rank's gathered arrays [world][rows][..] (sb_ep_gathered)
 *   sb_moe_experts_partial over the gathered rows: the routes that name this rank's experts, weighted sums per row
 *   sb_ep_combine   partial: this rank's sums for every rank's rows (fp32 [world][rows][hidden]); out = bf16(residual + the
 *                   ranks' sums for this rank's rows, added in rank order)
 * Windows are exchanged as CUDA IPC handles (SB_TP_HANDLE_BYTES each, rank order), as for sb_tp_connect. */
SB_API int sb_ep_create(uint32_t world, uint32_t rank, uint32_t rows, uint32_t hidden, uint32_t routes, void **out_group);
SB_API int sb_ep_destroy(void *group);
SB_API int sb_ep_export(void *group, void *handle_out /* SB_TP_HANDLE_BYTES */);
SB_API int sb_ep_connect(void *group, const void *handles /* [world][SB_TP_HANDLE_BYTES] */);
SB_API int sb_ep_gathered(void *group, void **out_rows, uint32_t **out_selected, float **out_weights);
SB_API int sb_ep_dispatch(void *stream, void *group, const void *rows, const uint32_t *selected, const float *weights);
SB_API int sb_ep_combine(void *stream, void *group, const float *partial, const void *residual, void *out);

SB_API int sb_target_create(const SbTargetConfig *config, void **out_target);
/* With tp_world > 1: the handle of this rank's exchange window, and the connection to all ranks' (sb_tp_export,
 * sb_tp_connect). A tensor-parallel target steps only after sb_target_tp_connect. */
SB_API int sb_target_tp_export(void *target, void *handle_out);
SB_API int sb_target_tp_connect(void *target, const void *handles);
/* This rank's share of the whole model's dimensions (equal to the configuration's without tensor parallelism). */
typedef struct SbTargetShare {
  uint32_t q_heads, q_head0, kv_heads, kv_head0, gdn_key_heads, gdn_key_head0, gdn_value_heads, gdn_value_head0;
  uint32_t intermediate, intermediate0, vocab, vocab0;
} SbTargetShare;
SB_API int sb_target_share(const SbTargetConfig *config, SbTargetShare *out_share);
SB_API int sb_target_destroy(void *target);
/* Device pointer and byte size of a tensor or buffer by name. Per layer (layer >= 0): attn_norm, ffn_norm,
 * in_proj, out_proj, ffn_gate, ffn_up, ffn_down, and for GDN layers ssm_ab, ssm_conv, ssm_a, ssm_dt_bias, ssm_norm,
 * state0/1, conv0/1, for attention layers q_norm, k_norm, kv_k, kv_v, kv_ks, kv_vs. Global (layer = -1):
 * token_embd, output_norm, output, logits, selected, results, hidden, tokens, uniforms, committed, penalty_words,
 * candidates, candidate_q, draws, constraint_masks, remaining (u32 [lanes]: the tokens each lane's request may still take,
 * 0xFFFFFFFF at creation; the step retains no more). The tensors a checkpoint fuses into in_proj are also reached one by one under their
 * GGUF stems, in the order of in_proj's rows: attn_q, attn_k, attn_v (attention layers), attn_qkv, attn_gate (GDN layers);
 * a target whose parts differ in format (sb_target_create_from_gguf) has only those, no in_proj. */
SB_API int sb_target_tensor(void *target, int layer, const char *name, void **out_dev, uint64_t *out_bytes);
/* The lane's sampling penalties (ops::SamplingPenalties, runtime/ops/Sampling.hpp:16-29; 1, 0, 0 switches them off): the
 * step then rewrites the logits in place before selection (sb_sample_penalize) from the table `penalty_words` (u32
 * [vocab], sb_target_tensor), which the host keeps current: the output's count of each token, bit 31 for the prompt's. */
SB_API int sb_target_set_penalties(void *target, float repetition, float presence, float frequency);
/* The end of the sampled rows' distribution (SamplingPolicy::minP / topK / topP, runtime/ops/Sampling.hpp:58-85: the tokens
 * min_p leaves, then the top_k most likely of those, then their top_p nucleus; 0 / 0 / 1 keep everything, the default).
 * Greedy steps (temperature 0) read none of the three. Vocabularies up to the limit of sb_sample_verify's filters. */
SB_API int sb_target_set_policy(void *target, float min_p, uint32_t top_k, float top_p);
/* A policy a lane (host array of SbTargetConfig.lanes entries; NULL: back to the step's temperature and sb_target_set_policy's
 * end for every lane): the lanes' steps then select each by its own temperature and end of the distribution, greedy and
 * sampled lanes side by side. The values live on the device and are read by the selection when it runs, so they can change
 * between steps without a new capture. Steps need uniforms while policies are set. */
SB_API int sb_target_set_lane_policies(void *target, const SbLanePolicy *policies_host);
/* The tokens that end a request (up to 16; NULL, 0: none): a retained stop token is the last token the step retains
 * (sb_accept's stop_tokens; the reference's StopTokens of Sampling::addAcceptance, runtime/ops/Sampling.hpp). */
SB_API int sb_target_set_stop_tokens(void *target, const uint32_t *stop_tokens_host, uint32_t n_stop);
/* The lane's admission (every lane's, with several): with `constrained` the step reads a constraint mask for every row from
 * the target's `constraint_masks` tensor (u32 [16 x lanes][ceil(vocab / 32)], sb_target_tensor), which the host (its grammar
 * or schema engine) fills before the step; excluded_host: up to 16 token ids no row selects (NULL, 0: none). The step then
 * runs sb_sample_admit on the logits before the penalties and the selection. */
SB_API int sb_target_set_admission(void *target, int constrained, const uint32_t *excluded_host, uint32_t n_excluded);
/* Seeded synthetic weights, a prefilled INT8 cache of `committed` tokens and random GDN state, written on the device. */
SB_API int sb_target_randomize(void *target, uint64_t seed, uint32_t committed);
/* Synthetic routing for measurements: with `given` != 0 every MoE block routes by the scores in the target's `moe_scores`
 * tensor (fp32 [rows of all lanes][experts], filled by the host, e.g. N(0, 1) as the benchmark's configuration states its
 * router logits) instead of its own router's; the router's projection still runs, into a buffer nothing reads. Random
 * weights do not make a router whose routes spread over the experts as a trained one's do. */
SB_API int sb_target_set_router_scores(void *target, int given);
/* Sets the lane's position (every lane's, with several) and clears the pending GDN rows. */
SB_API int sb_target_reset(void *target, uint32_t committed);
/* The same with a position per lane: committed_host holds SbTargetConfig.lanes words. */
SB_API int sb_target_reset_lanes(void *target, const uint32_t *committed_host);
/* One verify step over inputs already on the device (`tokens`, `uniforms` buffers of the target). */
SB_API int sb_target_step(void *target, void *stream, uint32_t rows, float temperature, uint32_t flags);
/* One verify step from host buffers: uploads the block's input tokens (row 0 the last accepted token, rows 1.. the
 * draft) and the uniforms, runs the step, downloads {retained, accepted, retained_rows, 0} and the retained tokens,
 * and waits. The results are checked before they are handed back (the reference's finalizeDecode,
 * runtime/model/Runtime.cpp:2943-2977): 1 <= retained <= rows, the retained rows a mask of that many rows with the anchor, accepted
 * below rows and at most retained, every retained token one of the vocabulary; SB_ERR_DEVICE otherwise (e.g. a row whose
 * admission left it no token selects 0xFFFFFFFF), with the outputs filled in for inspection. */
SB_API int sb_target_verify(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host, uint32_t rows,
                            float temperature, uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host);
/* sb_target_verify for a target of several lanes: tokens_host u32 [lanes][16] (a lane's block in its 16 slots, rows of them used),
 * uniforms_host fp32 [lanes][80] or NULL, out_tokens_host u32 [lanes][16] (a lane's retained tokens first), out_results_host
 * u32 [lanes][4] = {retained, accepted, retained_rows, 0} per lane. With SB_TARGET_TREE every lane's block is a tree: the
 * host has written the lanes' SplashTreeRow rows into the target's `tree` tensor ([lanes][16] rows) beforehand. */
SB_API int sb_target_verify_lanes(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host, uint32_t rows,
                                  float temperature, uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host);
/* sb_target_verify for a tree of draft tokens: tree_host holds `rows` SplashTreeRow entries {ancestors u32, parent u16,
 * depth u16}; sets SB_TARGET_TREE. out_tokens_host receives the accepted path's tokens. */
/* sb_target_verify_lanes for blocks of different lengths: lane_rows_host u32 [lanes], each 0..16, the rows of the lane's block
 * (the slots past them in tokens_host are ignored; a lane of 0 rows sits the step out: its position, cache and state stay).
 * The step runs max(lane_rows) row slots for every lane and selects, accepts and commits each lane by its own rows. */
SB_API int sb_target_verify_lanes_ragged(void *target, void *stream, const uint32_t *tokens_host, const float *uniforms_host,
                                         const uint32_t *lane_rows_host, float temperature, uint32_t flags, uint32_t *out_tokens_host,
                                         uint32_t *out_results_host);
SB_API int sb_target_verify_tree(void *target, void *stream, const uint32_t *tokens_host, const void *tree_host, const float *uniforms_host,
                                 uint32_t rows, float temperature, uint32_t flags, uint32_t *out_tokens_host, uint32_t *out_results_host);
/* Kernels one step launches, and the bytes its weights, cache and state stream (the roofline's numerator). */
/* The configuration the target was created with. */
SB_API int sb_target_config(void *target, SbTargetConfig *out_config);

/* ---- KV page pool ----
 * The pages of a target's INT8 cache as a pool its lanes draw from (the acquire / release of the reference's
 * engine::KvPool, runtime/engine/KvPool.hpp, for a fixed set of pages: no extents, no compaction, no shared prefixes). A lane
 * acquires the pages of the tokens it is about to hold (its position plus the step's rows) and releases them when its request
 * ends; SB_ERR_OOM, with nothing taken, when the pool cannot give them (the reference's KvPageAcquisition::failure).
 * sb_kv_pool_write_tables copies the lanes' page ids into the target's `page_table` (synchronous; between steps). A target
 * starts with every lane holding its own equal share of the pages; a pool made by sb_kv_pool_for_target takes all of them
 * over, with a lane's most pages the share it had. Host bookkeeping: everything but write_tables works without a device. */
SB_API int sb_kv_pool_create(uint32_t pages, uint32_t lanes, uint32_t lane_cap_pages, uint32_t page_tokens, void **out_pool);
SB_API int sb_kv_pool_for_target(void *target, void **out_pool);
SB_API int sb_kv_pool_destroy(void *pool);
SB_API int sb_kv_pool_acquire(void *pool, uint32_t lane, uint64_t tokens);
SB_API int sb_kv_pool_release(void *pool, uint32_t lane);
SB_API int sb_kv_pool_table(void *pool, uint32_t lane, const uint32_t **out_pages, uint32_t *out_count);
SB_API int sb_kv_pool_counts(void *pool, uint32_t *out_free, uint32_t *out_held);
SB_API int sb_kv_pool_write_tables(void *pool, void *target);

/* ---- prompt lookup ----
 * Proposals a request's own tokens make (the reference's LookupIndex, runtime/model/LookupProposals.hpp:17-66; step 1 of a
 * decode cycle, where the host proposes a lane's lookup chain): the index holds the request's tokens, its prompt and then
 * every token its steps retain, and after each append knows the match of the latest tokens - the earlier occurrence of
 * their longest suffix, its length counted up to 64 tokens, the most recent among those of that length, none shorter than
 * 3 tokens. sb_lookup_match gives the match's length (0: none) and the index of the earlier occurrence's last token;
 * sb_lookup_proposals copies up to `count` tokens that followed it (at most as far as the latest token): a verify block's
 * chain after its anchor. Host code: works without a device. */
SB_API int sb_lookup_create(void **out_index);
SB_API int sb_lookup_destroy(void *index);
SB_API int sb_lookup_append(void *index, const uint32_t *tokens, uint64_t count);
SB_API int sb_lookup_match(void *index, uint32_t *out_length, uint32_t *out_end);
SB_API int sb_lookup_proposals(void *index, uint32_t count, uint32_t *out_tokens, uint32_t *out_count);
SB_API int sb_lookup_size(void *index, uint64_t *out_tokens);
/* How a lookup token at `depth` (0: the first proposal after the anchor) compares with the draft's candidates (16 a proposal
 * position, the most likely first; `count` ids in all): 0 the most likely, 1 another candidate, 2 none of them, 3 unknown
 * (lookupAgreement, runtime/model/LookupProposals.cpp:170-178). */
SB_API int sb_lookup_agreement(uint32_t token, uint32_t depth, const uint32_t *candidates, uint64_t count, uint32_t *out_agreement);

/* ---- GGUF files ----
 * A reader of llama.cpp's GGUF container (version 3; the reference's runtime/model/GgufFile.hpp:23-141) over a read-only
 * mapping of the file, and the loader of a Qwen3.5 hybrid model (general.architecture qwen35 or qwen35moe) from it into a
 * target. The reader is host code: it works without a device. Tensor types are ggml's ids (0 F32, 1 F16, 8 Q8_0, 12 Q4_K,
 * 14 Q6_K, 30 BF16, ...); dims[0] is a row's length. Pointers handed out stay valid until sb_gguf_close. */
typedef struct SbGgufTensor {
  const char *name;
  uint32_t type, n_dims;
  uint64_t dims[4];  /* 1 past n_dims */
  const void *data;  /* host address of the tensor's bytes in the mapping */
  uint64_t bytes;
} SbGgufTensor;
SB_API int sb_gguf_open(const char *path, void **out_file);
/* The parts of a split GGUF in split order (gguf-split's parts: the keys split.no, split.count, split.tensors.count; the
 * first part holds the model's metadata) as one file: every part's tensors, the first part's metadata. A part given
 * alone, out of order or with parts missing is refused. */
SB_API int sb_gguf_open_parts(const char *const *paths, uint32_t count, void **out_file);
SB_API int sb_gguf_close(void *file);
SB_API int sb_gguf_tensor_count(void *file, uint64_t *out_count);
SB_API int sb_gguf_tensor(void *file, uint64_t index, SbGgufTensor *out);
SB_API int sb_gguf_find(void *file, const char *name, SbGgufTensor *out); /* SB_ERR_INVALID without such a tensor */
/* Scalar metadata by key: integers and booleans as unsigned (a negative one as its two's complement), floats (and
 * integers) as double, strings. SB_ERR_INVALID without such a key. */
SB_API int sb_gguf_meta_u64(void *file, const char *key, uint64_t *out);
SB_API int sb_gguf_meta_f64(void *file, const char *key, double *out);
SB_API int sb_gguf_meta_str(void *file, const char *key, const char **out);
/* A numeric array's values as doubles (arrays of up to 65536 numbers are kept; string arrays, e.g. the tokenizer's, are not). */
SB_API int sb_gguf_meta_array(void *file, const char *key, const double **out_values, uint64_t *out_count);
/* Fills the model's fields of *config from the file's metadata and tensors (the keys runtime/model/GgufImage.cpp:902-933
 * checks: block_count, embedding_length, attention.*, rope.*, full_attention_interval, ssm.*, expert_*,
 * feed_forward_length; the vocabulary from token_embd; fmt_* from the tensors' types; gated_attention from attn_q's rows;
 * tiled_heads = 1) and leaves the rest (page_tokens, kv_scale_f16, max_context, lanes, tp_*, ep_*) as the caller set them. */
SB_API int sb_gguf_target_config(void *file, SbTargetConfig *config);
/* The weight format (SB_FMT_*) of the rows behind a weight tensor's name of sb_target_tensor. */
SB_API int sb_target_tensor_format(void *target, int layer, const char *name, uint32_t *out_format);
/* A target made for the file and filled from it: the configuration of sb_gguf_target_config over *runtime (whose model
 * fields are ignored), and every projection tensor in the format the file stores it in, layer by layer - so a file that
 * mixes formats loads (llama.cpp's Q4_K_M keeps attn_v and half of the ffn_down tensors in Q6_K). Where the tensors fused
 * into a layer's input projection differ in format, the projection runs as one launch a tensor, each writing its columns
 * (the reference's fused column segments, runtime/ops/LinearGguf.cpp:25,78-86). ffn_gate and ffn_up of a layer share one
 * format; every type must be one a kernel reads (Q4_K, Q6_K, Q8_0). Not with tensor parallelism. */
SB_API int sb_target_create_from_gguf(void *file, const SbTargetConfig *runtime, void **out_target);
/* Copies the file's tensors into the target's (whole model on one GPU): names, shapes and conversions as
 * runtime/model/GgufImage.cpp:477-556 - attn_q / attn_k / attn_v (or attn_qkv and attn_gate) into the fused input
 * projection, ssm_beta / ssm_alpha into the fp32 gate rows, ssm_conv1d and ssm_dt.bias narrowed to bf16, the rows that
 * carry a value head gathered from llama.cpp's tiled head order into grouped order, stacked experts with the shared
 * expert last. A tensor whose type is not the format the target holds it in is refused by name (a target of sb_target_create
 * has one format for its projections, one for the down projections, one for the head and one for the embedding), so are
 * types no kernel here reads (e.g. Q5_K), and so is a file whose metadata differs from the target's configuration.
 * Synchronous. */
SB_API int sb_target_load_gguf(void *target, void *file);

SB_API int sb_target_stats(void *target, uint32_t rows, uint32_t *out_launches, uint64_t *out_weight_bytes, uint64_t *out_kv_bytes,
                           uint64_t *out_state_bytes);

#ifdef __cplusplus
}
#endif
#endif /* SPLASH_B200_H */
