// Down projection for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they
// run a layer: code inside a memory pool's own allocation callback, a plugin
// whose embedding runtime owns and pre-partitions the whole device heap, or a
// latency-critical decode loop that forbids allocator calls after start-up.
// The regular down projection splits the long reduction dimension over several
// CTAs and needs a caller-provided fp32 buffer for the partial sums.  This
// variant keeps those partial sums in a fixed array inside the library image
// instead and hands the caller only the finished [pairs, hidden] result.
#include "kernels.h"

namespace b200moe {
namespace {

// 2 Mi floats = 8 MiB, resident on every GPU that loads the library until the
// process exits.  Holds k-split partial sums: ksplit * pairs * hidden floats.
constexpr long long SCRATCH_FLOATS = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_down_scratch[SCRATCH_FLOATS];

// out[p, :] = sum over k-splits of the partial sums, added in split order, for
// the rows that belong to a local expert; rows past the last segment are zero.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(int ksplit, int pairs, int hidden, const int32_t* __restrict__ seg,
                       int experts, float* __restrict__ out) {
  const int valid = seg[experts];
  const long long n = static_cast<long long>(pairs) * hidden;
  const long long stride = n;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll) {
    float v = 0.f;
    if (i / hidden < valid) {
      for (int c = 0; c < ksplit; ++c) v += g_down_scratch[c * stride + i];
    }
    out[i] = v;
  }
}

// Device address of the scratch array for the current device.  In host code
// the symbol's name is only a handle; the address kernels can use comes from
// cudaGetSymbolAddress, once per device, with that device current.
float* scratch_ptr() {
  static float* ptrs[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
    set_error("down_noalloc: no usable current device");
    return nullptr;
  }
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_down_scratch);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaGetSymbolAddress(g_down_scratch)");
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_down_noalloc(const void* a, const int32_t* seg_offsets, int32_t pairs,
                                    int32_t max_segment, const b200moe_weight_t* down,
                                    float* d_out, void* stream) {
  B200_REQUIRE(down && seg_offsets, "down_noalloc: NULL argument");
  B200_REQUIRE(pairs >= 0, "down_noalloc: negative pair count");
  if (pairs == 0) return B200MOE_OK;
  B200_REQUIRE(a && d_out, "down_noalloc: NULL buffer");
  const int ks = stream_down_ksplit(down, pairs);
  const long long need = static_cast<long long>(ks) * pairs * down->rows;
  B200_REQUIRE(need <= SCRATCH_FLOATS,
               "down_noalloc: %d k-splits x %d pairs x %d hidden = %lld floats exceeds the "
               "built-in scratch of %lld floats (8 MiB); use b200moe_down with your own buffer",
               ks, pairs, down->rows, need, SCRATCH_FLOATS);
  float* scratch = scratch_ptr();
  if (scratch == nullptr) return B200MOE_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int rc = launch_stream_down(a, seg_offsets, pairs, max_segment, down, ks, scratch, st))
    return rc;
  const long long n = static_cast<long long>(pairs) * down->rows;
  const int blocks = static_cast<int>(n / 256 + 1 < 1184 ? n / 256 + 1 : 1184);
  reduce_partials_kernel<<<blocks, 256, 0, st>>>(ks, pairs, down->rows, seg_offsets, down->experts,
                                                 d_out);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}
