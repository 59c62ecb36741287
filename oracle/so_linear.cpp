// TEST INFRASTRUCTURE - CPU oracle, not part of the product library.
//
// Quantized linear Y = X W^T with the reference's numerics contract
// (runtime/metal/kernels/shared/gguf_linear.metal:113-130 staged tile,
// runtime/metal/kernels/common/gguf_tile.h:8-14 epilogues,
// runtime/metal/kernels/common/gguf_column_tile.h:25-68 summation order,
// runtime/metal/kernels/shared/gguf_linear.metal:38 one-pass gate/up,
// dev/tests/engine/GgufFormatReference.hpp:711-742 fp64 dot and projectionBound):
// bf16 inputs times exactly represented weight operands, fp32 accumulation, one rounding to the
// destination type after the epilogue.
//
//   so_linear_f64  fp64 dot products and the two error bounds of the reference's tests
//   so_linear      fp32 port in the column tile's order (chain of 32, then group sums in order);
//                  OpenMP over output columns; this is the timed host-CPU baseline
#include "so_common.h"

#include <omp.h>

#include <algorithm>
#include <vector>

SO_API uint64_t so_row_bytes(uint32_t f, uint32_t K);
SO_API int so_dequant(uint32_t f, const uint8_t *native, uint32_t rows, uint32_t K, float *out);

using namespace so;

// Sets the OpenMP thread count of every oracle routine (n > 0) and returns the count in force. A launcher may have
// exported OMP_NUM_THREADS=1 (torchrun does); the timed CPU baseline asks for the host's cores itself.
SO_API int so_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

// value[m*N+n] = sum_k x[m][k] w[n][k] in fp64 over the fp32 weight values;
// bound_exact = 2^-16 sum|x| max|w| (weights used unrounded), bound_staged adds 2^-11 sum|x w| +
// 2^-25 sum|x| (weights rounded once to half). Any of the three outputs may be null.
SO_API int so_linear_f64(uint32_t fmt, const uint8_t *W, uint32_t N, uint32_t K, const uint16_t *X, uint32_t M,
                         double *value, double *bound_exact, double *bound_staged) {
  const uint64_t rb = so_row_bytes(fmt, K);
  if (!rb) return -1;
  std::vector<float> xf(size_t(M) * K);
  std::vector<double> inputs(M, 0.0);
  for (uint32_t m = 0; m < M; ++m)
    for (uint32_t k = 0; k < K; ++k) {
      xf[size_t(m) * K + k] = bf2f(X[size_t(m) * K + k]);
      inputs[m] += std::fabs(double(xf[size_t(m) * K + k]));
    }
#pragma omp parallel
  {
    std::vector<float> w(K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < int64_t(N); ++n) {
      so_dequant(fmt, W + n * rb, 1, K, w.data());
      double largest = 0;
      for (uint32_t k = 0; k < K; ++k) largest = std::max(largest, double(std::fabs(w[k])));
      for (uint32_t m = 0; m < M; ++m) {
        const float *x = xf.data() + size_t(m) * K;
        double v = 0, mag = 0;
        for (uint32_t k = 0; k < K; ++k) {
          const double p = double(x[k]) * double(w[k]);
          v += p;
          mag += std::fabs(p);
        }
        const size_t at = size_t(m) * N + n;
        const double acc = std::ldexp(inputs[m] * largest, -16);
        if (value) value[at] = v;
        if (bound_exact) bound_exact[at] = acc;
        if (bound_staged) bound_staged[at] = acc + std::ldexp(mag, -11) + std::ldexp(inputs[m], -25);
      }
    }
  }
  return 0;
}

// Epilogues (SB_EPILOGUE_* of the product header): 0 none, 1 + residual, 2 up-with-gate
// (bf16(v) * silu(gate) with `aux` the gate values), 3 one-pass gate/up: W holds 2N rows, gate
// rows then up rows, output bf16(float(bf16(up)) * silu(float(bf16(gate)))).
// weight_mode 0: weights as their unrounded fp32 values; 1: rounded once to half (staged tile).
// out_f32 != 0 writes fp32 (the logits' destination), else bf16.
SO_API int so_linear(uint32_t fmt, const uint8_t *W, uint32_t N, uint32_t K, const uint16_t *X, uint32_t M,
                     uint32_t epilogue, const uint16_t *aux, uint32_t aux_stride, void *out, uint32_t out_stride,
                     uint32_t out_f32, uint32_t weight_mode) {
  const uint64_t rb = so_row_bytes(fmt, K);
  if (!rb || K % 32 || epilogue > 3) return -1;
  std::vector<float> xf(size_t(M) * K);
  for (size_t i = 0; i < xf.size(); ++i) xf[i] = bf2f(X[i]);
  auto dot = [&](const float *x, const float *w) {
    float total = 0.0f;
    for (uint32_t g = 0; g < K / 32; ++g) {
      float sum = 0.0f;
      for (uint32_t i = 0; i < 32; ++i) sum = sum + w[32 * g + i] * x[32 * g + i];
      total += sum;
    }
    return total;
  };
#pragma omp parallel
  {
    std::vector<float> w(K), w2(K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < int64_t(N); ++n) {
      so_dequant(fmt, W + n * rb, 1, K, w.data());
      if (epilogue == 3) so_dequant(fmt, W + (n + int64_t(N)) * rb, 1, K, w2.data());
      if (weight_mode == 1) {
        for (uint32_t k = 0; k < K; ++k) w[k] = rh(w[k]);
        if (epilogue == 3) for (uint32_t k = 0; k < K; ++k) w2[k] = rh(w2[k]);
      }
      for (uint32_t m = 0; m < M; ++m) {
        const float *x = xf.data() + size_t(m) * K;
        float v = dot(x, w.data());
        if (epilogue == 1) v += bf2f(aux[size_t(m) * aux_stride + n]);
        if (epilogue == 2) v = rbf(v) * silu(bf2f(aux[size_t(m) * aux_stride + n]));
        if (epilogue == 3) v = rbf(dot(x, w2.data())) * silu(rbf(v));
        if (out_f32) static_cast<float *>(out)[size_t(m) * out_stride + n] = v;
        else static_cast<uint16_t *>(out)[size_t(m) * out_stride + n] = f2bf(v);
      }
    }
  }
  return 0;
}
