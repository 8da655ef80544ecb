// Expert-parallel dispatch and combine by direct peer-to-peer stores over
// NVLink: no host synchronisation and no library collective per layer.
//
// Every rank maps every peer's buffers (symmetric allocation, same layout on all
// ranks).  Per layer:
//   publish   each rank writes its per-expert pair counts into row `rank` of
//             every peer's counts matrix [world][E]
//   barrier   flags with release/acquire at system scope; bounded spin
//   dispatch  one CTA per routed pair copies the token's normalised row into
//             the owning rank's receive buffer, at the position that groups
//             rows by (local expert, source rank) — the receiver needs no
//             regrouping pass, and its segment offsets follow from the counts
//   (grouped GEMMs on the receive buffer)
//   return    one CTA per received row adds the k-split partials, rounds to
//             bf16 and stores the row into the source rank's return buffer at the
//             pair's position in the source's own expert-sorted order
//   barrier, then the ordinary combine kernel at the source.
//
// Plain ld/st to peer memory only: no multimem, no TMA from peer memory.
#include "kernels.h"

namespace b200moe {
namespace {

constexpr int EP_MAX_WORLD = 16;
constexpr int EP_MAX_E = 64;

struct EpPtrs {
  int world, rank, el, E;
  int32_t* counts_all[EP_MAX_WORLD];  // [world][E] on each rank
  int32_t* flags[EP_MAX_WORLD];       // [world] on each rank
  uint4* recv_x[EP_MAX_WORLD];        // fp16 rows, grouped by (local expert, source)
  uint4* ret_y[EP_MAX_WORLD];         // bf16 rows in the source's sorted order
};

__global__ void ep_publish_kernel(EpPtrs p, const int32_t* __restrict__ counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.world * p.E) return;
  const int q = i / p.E, g = i % p.E;
  p.counts_all[q][p.rank * p.E + g] = counts[g];
}

// Signals every peer and waits for every peer.  Thread s talks to rank s.
// After the wait the caller's counts matrix is complete; thread 0 then derives
// the local segment offsets (rows per local expert summed over sources).
__global__ void __launch_bounds__(32)
ep_barrier_kernel(EpPtrs p, int epoch, int32_t* __restrict__ seg2, int32_t* status,
                  long long limit) {
  const int s = threadIdx.x;
  if (s < p.world) {
    __threadfence_system();
    int32_t* remote = p.flags[s] + p.rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int32_t* mine = p.flags[p.rank] + s;
    const long long t0 = clock64();
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v - epoch >= 0) break;
      if (clock64() - t0 > limit) {  // default ~2 s: a peer is gone; report, do not hang
        atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncwarp();
  if (s == 0 && seg2 != nullptr) {
    const int32_t* C = p.counts_all[p.rank];
    int run = 0;
    for (int e = 0; e < p.el; ++e) {
      seg2[e] = run;
      for (int src = 0; src < p.world; ++src) run += C[src * p.E + p.rank * p.el + e];
    }
    seg2[p.el] = run;
  }
}

// One CTA per expert-sorted pair of this rank.
__global__ void __launch_bounds__(128)
ep_dispatch_kernel(EpPtrs p, const uint4* __restrict__ xn, const int32_t* __restrict__ experts,
                   const int32_t* __restrict__ perm, const int32_t* __restrict__ seg, int top_k,
                   int vec_per_row, int kperm, int cap_rows, int32_t* status) {
  __shared__ int s_dst;
  const int i = blockIdx.x;
  const int pair = perm[i];
  if (threadIdx.x == 0) {
    const int g = experts[pair];
    const int q = g / p.el, e = g % p.el;
    const int32_t* C = p.counts_all[p.rank];
    int off = 0;
    for (int e2 = 0; e2 < e; ++e2)
      for (int src = 0; src < p.world; ++src) off += C[src * p.E + q * p.el + e2];
    for (int src = 0; src < p.rank; ++src) off += C[src * p.E + g];
    off += i - seg[g];
    if (off < 0 || off >= cap_rows) {
      atomicOr(status, DEV_ERR_BOUNDS);
      off = -1;
    }
    s_dst = off;
  }
  __syncthreads();
  if (s_dst < 0) return;
  const int g = experts[pair];
  const uint4* src = xn + static_cast<size_t>(pair / top_k) * vec_per_row;
  uint4* dst = p.recv_x[g / p.el] + static_cast<size_t>(s_dst) * vec_per_row;
  for (int j = threadIdx.x; j < vec_per_row; j += blockDim.x) {
    uint4 v = src[j];
    if (kperm) {
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);
      o.y = __byte_perm(v.x, v.z, 0x7632);
      o.z = __byte_perm(v.y, v.w, 0x5410);
      o.w = __byte_perm(v.y, v.w, 0x7632);
      v = o;
    }
    dst[j] = v;
  }
}

// One CTA per row of the receive buffer (grid = capacity; rows past the last
// segment exit).  d_rows: fp32 [ksplit][cap_rows][d].
__global__ void __launch_bounds__(128)
ep_return_kernel(EpPtrs p, const float* __restrict__ d_rows, int ksplit, int cap_rows, int d,
                 const int32_t* __restrict__ seg2, int ret_rows, int32_t* status) {
  __shared__ int s_src, s_dst;
  const int i = blockIdx.x;
  if (i >= seg2[p.el]) return;
  if (threadIdx.x == 0) {
    const int32_t* C = p.counts_all[p.rank];
    int e = 0;
    while (i >= seg2[e + 1]) ++e;
    const int g = p.rank * p.el + e;
    int j = i - seg2[e], src = 0;
    while (src < p.world - 1 && j >= C[src * p.E + g]) { j -= C[src * p.E + g]; ++src; }
    int off = 0;
    for (int g2 = 0; g2 < g; ++g2) off += C[src * p.E + g2];
    off += j;
    if (off < 0 || off >= ret_rows) {
      atomicOr(status, DEV_ERR_BOUNDS);
      off = -1;
    }
    s_src = src;
    s_dst = off;
  }
  __syncthreads();
  if (s_dst < 0) return;
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(p.ret_y[s_src]) +
                        static_cast<size_t>(s_dst) * (d / 2);
  const size_t stride = static_cast<size_t>(cap_rows) * d;
  const float* row = d_rows + static_cast<size_t>(i) * d;
  for (int j = threadIdx.x; j < d / 2; j += blockDim.x) {
    float a = 0.f, b = 0.f;
    for (int c = 0; c < ksplit; ++c) {
      const float2 v = *reinterpret_cast<const float2*>(row + c * stride + 2 * j);
      a += v.x;
      b += v.y;
    }
    dst[j] = __floats2bfloat162_rn(a, b);
  }
}

// spin limit of the cross-GPU barrier in clock ticks (b200moe_set_wait_limit)
long long g_barrier_ticks = 1ll << 32;

int fill(EpPtrs* p, const b200moe_ep_t* ep) {
  B200_REQUIRE(ep != nullptr, "ep: NULL descriptor");
  B200_REQUIRE(ep->world >= 1 && ep->world <= EP_MAX_WORLD && ep->rank >= 0 && ep->rank < ep->world,
               "ep: world %d / rank %d out of range", ep->world, ep->rank);
  B200_REQUIRE(ep->experts_local >= 1 && ep->experts_local * ep->world <= EP_MAX_E,
               "ep: %d local experts x %d ranks out of range", ep->experts_local, ep->world);
  p->world = ep->world; p->rank = ep->rank; p->el = ep->experts_local;
  p->E = ep->experts_local * ep->world;
  for (int i = 0; i < ep->world; ++i) {
    B200_REQUIRE(ep->counts_all[i] && ep->flags[i] && ep->recv_x[i] && ep->ret_y[i],
                 "ep: missing peer pointer for rank %d", i);
    p->counts_all[i] = static_cast<int32_t*>(ep->counts_all[i]);
    p->flags[i] = static_cast<int32_t*>(ep->flags[i]);
    p->recv_x[i] = static_cast<uint4*>(ep->recv_x[i]);
    p->ret_y[i] = static_cast<uint4*>(ep->ret_y[i]);
  }
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_ep_publish_counts(const b200moe_ep_t* ep, const int32_t* counts, void* stream) {
  EpPtrs p;
  if (int rc = fill(&p, ep)) return rc;
  B200_REQUIRE(counts != nullptr, "ep_publish_counts: NULL counts");
  const int n = p.world * p.E;
  ep_publish_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(p, counts);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_set_wait_limit(int64_t clock_ticks) {
  B200_REQUIRE(clock_ticks >= 0, "set_wait_limit: negative tick count");
  g_barrier_ticks = clock_ticks == 0 ? (1ll << 32) : static_cast<long long>(clock_ticks);
  return B200MOE_OK;
}

int b200moe_ep_barrier(const b200moe_ep_t* ep, int32_t epoch, int32_t* seg2_out, void* stream) {
  EpPtrs p;
  if (int rc = fill(&p, ep)) return rc;
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, epoch, seg2_out, status,
                                                                   g_barrier_ticks);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_ep_dispatch(const b200moe_ep_t* ep, const void* xn, const int32_t* experts,
                        const int32_t* perm, const int32_t* seg_offsets, int32_t pairs,
                        int32_t top_k, int32_t hidden, int32_t kperm, int32_t cap_rows,
                        void* stream) {
  EpPtrs p;
  if (int rc = fill(&p, ep)) return rc;
  B200_REQUIRE(hidden % 8 == 0 && top_k >= 1 && cap_rows >= 0, "ep_dispatch: bad sizes");
  if (pairs == 0) return B200MOE_OK;
  B200_REQUIRE(xn && experts && perm && seg_offsets, "ep_dispatch: NULL buffer");
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  ep_dispatch_kernel<<<pairs, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      p, static_cast<const uint4*>(xn), experts, perm, seg_offsets, top_k, hidden / 8, kperm,
      cap_rows, status);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_ep_return(const b200moe_ep_t* ep, const float* d_rows, int32_t ksplit,
                      int32_t cap_rows, const int32_t* seg2, int32_t hidden, int32_t ret_rows,
                      void* stream) {
  EpPtrs p;
  if (int rc = fill(&p, ep)) return rc;
  B200_REQUIRE(hidden % 2 == 0 && ksplit >= 1 && cap_rows >= 0, "ep_return: bad sizes");
  if (cap_rows == 0) return B200MOE_OK;
  B200_REQUIRE(d_rows && seg2, "ep_return: NULL buffer");
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  ep_return_kernel<<<cap_rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      p, d_rows, ksplit, cap_rows, hidden, seg2, ret_rows, status);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

}  // extern "C"
