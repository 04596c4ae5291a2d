// Declarations shared by the translation units of libthinfer_nvfp4.so (not part of the ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <tuple>
#include <utility>

namespace tnf {

// Launch with programmatic dependent launch allowed: the kernel's prologue and CTA scheduling may
// overlap the tail of the previous kernel in the stream. Only for kernels that call pdl_wait()
// before touching global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// 512-byte scale atoms along K per 128-row block: ceil(K/64) rounded up to a multiple of 4,
// so that a 256-element K tile always reads four whole, contiguous atoms.
__host__ __device__ inline uint32_t sf_k_atoms(uint32_t k) { return (((k + 63u) / 64u) + 3u) & ~3u; }
inline uint64_t sf_device_bytes(uint32_t rows, uint32_t k) {
  return uint64_t((rows + 127u) / 128u) * sf_k_atoms(k) * 512ull;
}

constexpr int kMaxPeers = 8;
constexpr int kMaxDevices = 64;

// Diagnostic variant of the library (clock64 traces, "skip this part" switches, kernel-selection
// overrides from the environment): compiled only with -DTNF_GEMM_DIAG. In the default build every
// `if (kDiag && ...)` below is removed by the compiler and the library reads no environment variable.
#ifdef TNF_GEMM_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif

// Function attributes (dynamic shared memory opt-in, carve-out) belong to a device, not to the
// process: launchers keep one of these per kernel and set the attributes on first use per device.
struct PerDeviceOnce {
  bool done[kMaxDevices] = {};
  // index of the current device, or -1 when it has been seen before (or cannot be tracked)
  int first_use() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;  // untracked: set every time
    if (done[dev]) return -1;
    done[dev] = true;
    return dev;
  }
};

// Default upper bound of a device-side mbarrier wait, in SM cycles (about two seconds).
constexpr long long kDefaultWaitLimitCycles = 4000000000ll;

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
  uint32_t full_tiles;         // pair kernel: tiles [0, full_tiles) run whole; each later one as two 128-column halves
  uint8_t* q_codes;            // optional NVFP4 copy of the output: codes [m, n/2] ...
  uint8_t* q_scales;           // ... and device-layout scales of an [m, n] operand
  float q_global, q_inv_t;     // its per-tensor scale g and 1/(6g)
  uint32_t q_k_atoms;          // sf_k_atoms(n)
  uint16_t* out_mc;            // multicast alias of out[0] (null: plain stores); with it every store of the epilogue
  uint8_t* q_codes_mc;         //   (bf16 rows, NVFP4 codes, scale words) goes out as multimem.st and lands on
  uint8_t* q_scales_mc;        //   every rank of the group, this one included
  uint32_t dense;              // dense-activation arm: A is bf16 [m,k], W the exact bf16 image of code x block scale
                               // [n,k]; no scale factors, tcgen05.mma kind::f16 (pair kernel only)
  uint32_t swiglu;             // pairwise gating epilogue: out[m, j] = silu(v[2j]) * v[2j+1], n/2 output columns
  uint32_t store_bf16;         // 0: skip the bf16 store
  uint32_t* status;            // device status word
  long long wait_limit;        // SM cycles after which a device-side wait gives up (0 = kDefaultWaitLimitCycles)
  uint32_t stall;              // self-test: the producer issues no loads, so the first wait on a loaded stage runs out
  uint32_t diag;               // diagnostic builds only (kDiag), bits from TNF_GEMM_DIAG: 1 no output stores,
                               // 2 scale copies only on the first K tile, 4 no MMA, 8 no operand loads,
                               // 16 record clock64 stamps of the first K tiles of pair 0 into `trace`
  unsigned long long* trace;   // 4 stamps per K tile (diag bit 16), 256 K tiles
};

cudaError_t launch_amax(const void* x, int dtype, uint64_t n, uint32_t* amax_bits, cudaStream_t s);
cudaError_t launch_global_scale(const uint32_t* amax_bits, float* g, cudaStream_t s);
cudaError_t launch_quantize(const void* src, int dtype, uint32_t rows, uint32_t k, const float* g_ptr, float g_val,
                            uint8_t* codes, uint8_t* scales, bool device_layout, cudaStream_t s);
cudaError_t launch_multicast_copy(const uint8_t* src, uint8_t* dst_mc, uint64_t bytes, int sm_count, cudaStream_t s);
cudaError_t launch_dequant_dense(const uint8_t* codes, const uint8_t* scales_device, uint32_t n, uint32_t k, uint16_t* out_bf16,
                                 cudaStream_t s);
cudaError_t launch_scales_to_device(const uint8_t* in, uint32_t rows, uint32_t k, uint8_t* out, cudaStream_t s);

// tcgen05 GEMM. a_codes [m, k/2], w_codes [n, k/2]; tensor maps are built (and cached) by the caller.
cudaError_t launch_gemm_nvfp4(const CUtensorMap& map_a, const CUtensorMap& map_w, const GemmParams& p, int sm_count,
                              cudaStream_t s);
// CTA-pair kernel (256x256 tiles, large M). out_maps[i] covers destination i's [m, n] window.
cudaError_t launch_gemm_nvfp4_pair(const CUtensorMap& map_a, const CUtensorMap& map_w, const CUtensorMap& map_sfa,
                                   const CUtensorMap& map_sfb, const CUtensorMap* out_maps, const GemmParams& p,
                                   int sm_count, cudaStream_t s);
// Skinny-M kernel (M <= 8): activation quantiser + weight streaming on the CUDA cores in one launch.
// Skinny-M on the tensor cores with the operands swapped (M <= 16, one launch, quantiser in the prologue); map_w is the
// weight's codes as [n, k/2] bytes with a {128 B, 128 rows} box and 128-byte swizzle.
bool skinny_tc_capable(uint32_t m, uint32_t n, uint32_t k);  // the tensor-core skinny kernel can run this shape
bool skinny_tc_applies(uint32_t m, uint32_t n, uint32_t k);  // ... and is the faster path for it
cudaError_t launch_skinny_tc(const CUtensorMap& map_w, const void* a_bf16, float a_global, const GemmParams& p, cudaStream_t s);
bool gemv_applies(uint32_t m, uint32_t n, uint32_t k);
cudaError_t launch_gemv_nvfp4(const void* a_bf16, float a_global, const uint8_t* w_codes, const GemmParams& p, cudaStream_t s);
bool gemm_use_pair(uint32_t m, uint32_t n, uint32_t k);
uint32_t gemm_pair_kblocks();  // 64-element K blocks per pipeline stage of the pair kernel (2 or 4): sets the TMA boxes

// 2-D tensor map description (dim0 is the contiguous one); all maps are built through this.
struct MapSpec {
  const void* base;
  uint32_t elem_bytes;   // 1 (uint8) or 2 (bf16)
  uint64_t dim0, dim1;   // extents in elements
  uint64_t stride1;      // bytes between rows
  uint32_t box0, box1;   // box in elements
  uint32_t swizzle128;   // swizzle span in bytes: 128, 64 or 0 (none); 1 also means 128
  bool operator<(const MapSpec& o) const {
    return std::tie(base, elem_bytes, dim0, dim1, stride1, box0, box1, swizzle128) <
           std::tie(o.base, o.elem_bytes, o.dim0, o.dim1, o.stride1, o.box0, o.box1, o.swizzle128);
  }
};
int make_tensor_map(CUtensorMap* out, const MapSpec& spec);
uint32_t gemm_tile_n(uint32_t m, uint32_t n);  // tile width the 1-CTA launcher will pick for this n (for the map of W)

}  // namespace tnf
