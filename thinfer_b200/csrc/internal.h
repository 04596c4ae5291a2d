// Declarations shared by the translation units of libthinfer_nvfp4.so (not part of the ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>

namespace tnf {

// 512-byte scale atoms along K per 128-row block: ceil(K/64) rounded up to a multiple of 4,
// so that a 256-element K tile always reads four whole, contiguous atoms.
__host__ __device__ inline uint32_t sf_k_atoms(uint32_t k) { return (((k + 63u) / 64u) + 3u) & ~3u; }
inline uint64_t sf_device_bytes(uint32_t rows, uint32_t k) {
  return uint64_t((rows + 127u) / 128u) * sf_k_atoms(k) * 512ull;
}

constexpr int kMaxPeers = 8;

// Device-side status word values (first failure wins).
enum : uint32_t {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,
  kStatusMmaTimeout = 2,
  kStatusEpilogueTimeout = 3,
  kStatusAccEmptyTimeout = 4
};

struct GemmParams {
  uint32_t m, n, k;
  uint32_t k_atoms;            // sf_k_atoms(k)
  float alpha;                 // a_global * w_global
  const uint8_t* sfa;          // device-layout scales of A
  const uint8_t* sfb;          // device-layout scales of W
  const uint16_t* bias;        // [n] bf16 or null
  const uint16_t* gate;        // [n] bf16 or null
  const uint16_t* residual;    // [m, n] bf16 or null (with gate)
  uint16_t* out[kMaxPeers];    // out[0] is local; the rest are peer windows
  uint32_t n_out;              // number of destinations (>= 1)
  uint32_t ldo, n_offset;
  uint32_t act, chain;
  uint32_t tiles_m, tiles_n;
  uint32_t* status;            // device status word
  uint32_t diag;               // diagnostic bits from TNF_GEMM_DIAG (0 in normal use): 1 no output stores,
                               // 2 scale copies only on the first K tile, 4 no MMA, 8 no operand loads
};

cudaError_t launch_amax(const void* x, int dtype, uint64_t n, uint32_t* amax_bits, cudaStream_t s);
cudaError_t launch_global_scale(const uint32_t* amax_bits, float* g, cudaStream_t s);
cudaError_t launch_quantize(const void* src, int dtype, uint32_t rows, uint32_t k, const float* g_ptr, float g_val,
                            uint8_t* codes, uint8_t* scales, bool device_layout, cudaStream_t s);
cudaError_t launch_scales_to_device(const uint8_t* in, uint32_t rows, uint32_t k, uint8_t* out, cudaStream_t s);

// tcgen05 GEMM. a_codes [m, k/2], w_codes [n, k/2]; tensor maps are built (and cached) by the caller.
cudaError_t launch_gemm_nvfp4(const CUtensorMap& map_a, const CUtensorMap& map_w, const GemmParams& p, int sm_count,
                              cudaStream_t s);
// Tensor map over packed E2M1 codes viewed as bytes [rows, k/2], box {128 bytes, box_rows}, 128-byte swizzle.
int make_codes_tensor_map(CUtensorMap* out, const void* base, uint32_t rows, uint32_t k, uint32_t box_rows);
uint32_t gemm_tile_n(uint32_t n);  // tile width the launcher will pick for this n (for the map of W)

}  // namespace tnf
