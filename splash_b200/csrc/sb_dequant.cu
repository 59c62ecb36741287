// Device dequantization of GGUF native rows to fp32, or to fp16 rounded once: the values the
// reference's dequantization test demands bit for bit (dev/tests/engine/gguf_dequant_test.mm:50-56;
// CPU twin dev/tests/engine/GgufFormatReference.hpp:370-381,418-432,453-458; kernel form
// runtime/metal/kernels/common/gguf_staged.h:11-17). Every product below is exact in fp32, so the
// single rounding of d*sc*q - dmin*mn is the same whether it is written as a chain or as an fma.
#include <algorithm>

#include "sb_dequant.cuh"

namespace sb {

// One thread per weight; grid-stride over rows * k.
__global__ void dequant_kernel(uint32_t format, const uint8_t *w, uint64_t row_bytes, uint32_t rows, uint32_t k,
                               void *out, uint32_t out_f16) {
  const uint64_t total = uint64_t(rows) * k;
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
    const uint32_t r = uint32_t(i / k), c = uint32_t(i % k);
    const uint8_t *row = w + r * row_bytes;
    const float v = weight_value(format, row, c);
    if (out_f16) static_cast<__half *>(out)[i] = __float2half_rn(v);
    else static_cast<float *>(out)[i] = v;
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_dequant(void *stream, uint32_t format, const void *weights_dev, uint32_t rows, uint32_t k,
                          void *out_dev, uint32_t out_f16) {
  SB_NEED_DEVICE();
  SB_REQUIRE(weights_dev && out_dev, "sb_dequant: null pointer");
  SB_REQUIRE(format == SB_FMT_Q4K || format == SB_FMT_Q6K || format == SB_FMT_Q80 || format == SB_FMT_NVFP4,
             "sb_dequant: unsupported format %u", format);
  const uint64_t rb = sb_row_bytes(format, k);
  SB_REQUIRE(rb != 0 && rows != 0, "sb_dequant: k = %u is not whole blocks of format %u, or no rows", k, format);
  const uint64_t total = uint64_t(rows) * k;
  const uint32_t blocks = uint32_t(std::min<uint64_t>((total + 255) / 256, uint64_t(ctx().sm_count) * 16));
  dequant_kernel<<<blocks, 256, 0, as_stream(stream)>>>(format, static_cast<const uint8_t *>(weights_dev), rb, rows, k,
                                                       out_dev, out_f16);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
