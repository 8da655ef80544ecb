// Router, route plan, row permutation, combine, reference dequantisation and
// GGUF block unpacking.  All HBM-bound or latency-bound helpers around the two
// expert-GEMM kernels.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace b200moe {

// ------------------------------------------------------------------ router
// One warp per token.  RMS norm in fp32 (x * 1/sqrt(mean(x^2)+eps), then the
// norm weight), router logits from the fp32 normalised row, fp32 softmax,
// top-k by descending probability (ties: lowest expert id) and renormalised
// gates.  The normalised row is written as fp16 for the expert products.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

constexpr int ROUTER_WARPS = 8;
constexpr int MAX_EXPERTS = 64;
constexpr int MAX_TOPK = 8;

template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_kernel(const T* __restrict__ h, int tokens, int d, int E, int k, float eps,
              const float* __restrict__ norm_w, const float* __restrict__ rw,
              const float* __restrict__ rb, __half* __restrict__ xn_out,
              int32_t* __restrict__ experts_out, float* __restrict__ gates_out) {
  __shared__ float s_logit[ROUTER_WARPS][MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTER_WARPS + warp;
  if (t >= tokens) return;
  const T* row = h + static_cast<size_t>(t) * d;

  float ss = 0.f;
  for (int j = lane * 8; j < d; j += 256) {
    float v[8];
    load8<T>(row + j, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);

  for (int e0 = 0; e0 < E; e0 += 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = lane * 8; j < d; j += 256) {
      float v[8], w[8];
      load8<T>(row + j, v);
      load8<float>(norm_w + j, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = w[i] * (v[i] * rstd);
      if (e0 == 0) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          packed[i] = h2_as_u32(__halves2half2(to_half_sat(v[2 * i]), to_half_sat(v[2 * i + 1])));
        *reinterpret_cast<uint4*>(xn_out + static_cast<size_t>(t) * d + j) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (e0 + e < E) {
          float r[8];
          load8<float>(rw + static_cast<size_t>(e0 + e) * d + j, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[e] = fmaf(v[i], r[i], acc[e]);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
      if (lane == 0 && e0 + e < E) s_logit[warp][e0 + e] = acc[e] + (rb ? rb[e0 + e] : 0.f);
    }
  }
  __syncwarp();

  // softmax over E <= 64: lane owns experts lane and lane+32
  const float NEG = -INFINITY;
  float l0 = lane < E ? s_logit[warp][lane] : NEG;
  float l1 = lane + 32 < E ? s_logit[warp][lane + 32] : NEG;
  float mx = fmaxf(l0, l1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float p0 = lane < E ? expf(l0 - mx) : 0.f;
  float p1 = lane + 32 < E ? expf(l1 - mx) : 0.f;
  float sum = p0 + p1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  p0 = lane < E ? p0 / sum : -1.f;
  p1 = lane + 32 < E ? p1 / sum : -1.f;

  float sel_p[MAX_TOPK];
  int sel_i[MAX_TOPK];
  float gsum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) {
    if (i < k) {
      float bp = p0;
      int bi = lane;
      if (p1 > bp) { bp = p1; bi = lane + 32; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float op = __shfl_xor_sync(0xffffffffu, bp, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (op > bp || (op == bp && oi < bi)) { bp = op; bi = oi; }
      }
      sel_p[i] = bp;
      sel_i[i] = bi;
      gsum += bp;
      if (bi == lane) p0 = -1.f;
      if (bi == lane + 32) p1 = -1.f;
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < MAX_TOPK; ++i) {
      if (i < k) {
        experts_out[static_cast<size_t>(t) * k + i] = sel_i[i];
        gates_out[static_cast<size_t>(t) * k + i] = sel_p[i] / gsum;
      }
    }
  }
}

// Softmax over the logits of one token held in shared memory, top-k and gate
// renormalisation by one warp (shared by both router kernels).
__device__ __forceinline__ void router_select(const float* logit, int lane, int E, int k,
                                              int32_t* experts_out, float* gates_out) {
  const float NEG = -INFINITY;
  float l0 = lane < E ? logit[lane] : NEG;
  float l1 = lane + 32 < E ? logit[lane + 32] : NEG;
  float mx = fmaxf(l0, l1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float p0 = lane < E ? expf(l0 - mx) : 0.f;
  float p1 = lane + 32 < E ? expf(l1 - mx) : 0.f;
  float sum = p0 + p1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  p0 = lane < E ? p0 / sum : -1.f;
  p1 = lane + 32 < E ? p1 / sum : -1.f;
  float sel_p[MAX_TOPK];
  int sel_i[MAX_TOPK];
  float gsum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) {
    if (i < k) {
      float bp = p0;
      int bi = lane;
      if (p1 > bp) { bp = p1; bi = lane + 32; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float op = __shfl_xor_sync(0xffffffffu, bp, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (op > bp || (op == bp && oi < bi)) { bp = op; bi = oi; }
      }
      sel_p[i] = bp;
      sel_i[i] = bi;
      gsum += bp;
      if (bi == lane) p0 = -1.f;
      if (bi == lane + 32) p1 = -1.f;
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < MAX_TOPK; ++i) {
      if (i < k) {
        experts_out[i] = sel_i[i];
        gates_out[i] = sel_p[i] / gsum;
      }
    }
  }
}

// Prefill: persistent CTAs with the router weight and the norm weight resident
// in shared memory.  With one token per warp reading them from global memory,
// every warp streams the whole router weight (E x d fp32) out of L2 for itself:
// 4096 tokens x 128 KB for a Mixtral layer, which is what that kernel's time is.
// Here a CTA loads them once (E*d*4 + d*4 bytes, up to ~220 KB) and its eight
// warps walk over the tokens; only the activations move through HBM.  Per token
// the operations and their order are those of router_kernel, so experts and gates
// are bit-identical to it.
//
// Shared layout: element j = 256*it + 8*lane + 4*hf + i of a vector is stored at
// ((it*2 + hf)*32 + lane)*4 + i, so that the two 16-byte reads a lane makes per
// step are conflict-free.
constexpr int RS_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(RS_WARPS * 32)
router_smem_kernel(const T* __restrict__ h, int tokens, int d, int E, int k, float eps,
                   const float* __restrict__ norm_w, const float* __restrict__ rw,
                   const float* __restrict__ rb, __half* __restrict__ xn_out,
                   int32_t* __restrict__ experts_out, float* __restrict__ gates_out) {
  extern __shared__ float s_dyn[];
  float* s_w = s_dyn;                       // [E][d] in the layout above
  float* s_n = s_dyn + static_cast<size_t>(E) * d;  // [d]
  float* s_logit = s_n + d;                 // [RS_WARPS][MAX_EXPERTS]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto slot = [](int j) { return (((j >> 8) * 2 + ((j >> 2) & 1)) * 32 + ((j >> 3) & 31)) * 4 + (j & 3); };
  for (int idx = threadIdx.x * 4; idx < E * d; idx += RS_WARPS * 32 * 4) {
    const int e = idx / d, j = idx - e * d;
    *reinterpret_cast<float4*>(s_w + static_cast<size_t>(e) * d + slot(j)) =
        *reinterpret_cast<const float4*>(rw + idx);
  }
  for (int j = threadIdx.x * 4; j < d; j += RS_WARPS * 32 * 4)
    *reinterpret_cast<float4*>(s_n + slot(j)) = *reinterpret_cast<const float4*>(norm_w + j);
  __syncthreads();

  for (int t = blockIdx.x * RS_WARPS + warp; t < tokens; t += gridDim.x * RS_WARPS) {
    const T* row = h + static_cast<size_t>(t) * d;
    float ss = 0.f;
    for (int j = lane * 8; j < d; j += 256) {
      float v[8];
      load8<T>(row + j, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);

    for (int e0 = 0; e0 < E; e0 += 8) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = lane * 8; j < d; j += 256) {
        float v[8], w[8];
        load8<T>(row + j, v);  // second pass: the row is in L1/L2
        const int base = ((j >> 8) * 2 * 32 + lane) * 4;  // hf = 0; hf = 1 is 128 floats further
        {
          const float4 a = *reinterpret_cast<const float4*>(s_n + base);
          const float4 b = *reinterpret_cast<const float4*>(s_n + base + 128);
          w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
          w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = w[i] * (v[i] * rstd);
        if (e0 == 0) {
          uint32_t packed[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            packed[i] = h2_as_u32(__halves2half2(to_half_sat(v[2 * i]), to_half_sat(v[2 * i + 1])));
          *reinterpret_cast<uint4*>(xn_out + static_cast<size_t>(t) * d + j) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (e0 + e < E) {
            const float* wr = s_w + static_cast<size_t>(e0 + e) * d + base;
            const float4 a = *reinterpret_cast<const float4*>(wr);
            const float4 b = *reinterpret_cast<const float4*>(wr + 128);
            const float r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[e] = fmaf(v[i], r[i], acc[e]);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
        if (lane == 0 && e0 + e < E)
          s_logit[warp * MAX_EXPERTS + e0 + e] = acc[e] + (rb ? rb[e0 + e] : 0.f);
      }
    }
    __syncwarp();
    router_select(s_logit + warp * MAX_EXPERTS, lane, E, k, experts_out + static_cast<size_t>(t) * k,
                  gates_out + static_cast<size_t>(t) * k);
    __syncwarp();  // the logits are rewritten for the warp's next token
  }
}

// The same kernel for bf16 activations with the token's row held in registers:
// all of a row's loads are issued at once (one memory latency per token instead
// of one per loop iteration) and, with PREFETCH, the next token's row is already
// in flight while this one is being routed.  Arithmetic and its order are
// unchanged.  MAXIT >= hidden / 256 (16: hidden up to 4096).
template <int MAXIT, bool PREFETCH>
__global__ void __launch_bounds__(RS_WARPS * 32)
router_smem_bf16_kernel(const __nv_bfloat16* __restrict__ h, int tokens, int d, int E, int k, float eps,
                        const float* __restrict__ norm_w, const float* __restrict__ rw,
                        const float* __restrict__ rb, __half* __restrict__ xn_out,
                        int32_t* __restrict__ experts_out, float* __restrict__ gates_out) {
  extern __shared__ float s_dyn[];
  float* s_w = s_dyn;
  float* s_n = s_dyn + static_cast<size_t>(E) * d;
  float* s_logit = s_n + d;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nit = d >> 8;
  const int stride = gridDim.x * RS_WARPS;
  int t = blockIdx.x * RS_WARPS + warp;
  uint4 cur[MAXIT], nxt[PREFETCH ? MAXIT : 1];
#define B200_LOAD_ROW(dst, tok)                                                              \
  {                                                                                          \
    const uint4* row_ = reinterpret_cast<const uint4*>(h + static_cast<size_t>(tok) * d) + lane; \
    _Pragma("unroll") for (int it = 0; it < MAXIT; ++it) if (it < nit) dst[it] = row_[it * 32];  \
  }
  if (t < tokens) B200_LOAD_ROW(cur, t);  // in flight while the weights are staged
  auto slot = [](int j) { return (((j >> 8) * 2 + ((j >> 2) & 1)) * 32 + ((j >> 3) & 31)) * 4 + (j & 3); };
  for (int idx = threadIdx.x * 4; idx < E * d; idx += RS_WARPS * 32 * 4) {
    const int e = idx / d, j = idx - e * d;
    *reinterpret_cast<float4*>(s_w + static_cast<size_t>(e) * d + slot(j)) =
        *reinterpret_cast<const float4*>(rw + idx);
  }
  for (int j = threadIdx.x * 4; j < d; j += RS_WARPS * 32 * 4)
    *reinterpret_cast<float4*>(s_n + slot(j)) = *reinterpret_cast<const float4*>(norm_w + j);
  __syncthreads();

  auto unpack = [](const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  };

  for (; t < tokens; t += stride) {
    if constexpr (PREFETCH) {
      if (t + stride < tokens) B200_LOAD_ROW(nxt, t + stride);
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXIT; ++it) {
      if (it < nit) {
        float v[8];
        unpack(cur[it], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);

    for (int e0 = 0; e0 < E; e0 += 8) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
      for (int it = 0; it < MAXIT; ++it) {
        if (it < nit) {
          float v[8], w[8];
          unpack(cur[it], v);
          const int base = (it * 2 * 32 + lane) * 4;
          {
            const float4 a = *reinterpret_cast<const float4*>(s_n + base);
            const float4 b = *reinterpret_cast<const float4*>(s_n + base + 128);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = w[i] * (v[i] * rstd);
          if (e0 == 0) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              packed[i] = h2_as_u32(__halves2half2(to_half_sat(v[2 * i]), to_half_sat(v[2 * i + 1])));
            *reinterpret_cast<uint4*>(xn_out + static_cast<size_t>(t) * d + it * 256 + lane * 8) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (e0 + e < E) {
              const float* wr = s_w + static_cast<size_t>(e0 + e) * d + base;
              const float4 a = *reinterpret_cast<const float4*>(wr);
              const float4 b = *reinterpret_cast<const float4*>(wr + 128);
              const float r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[e] = fmaf(v[i], r[i], acc[e]);
            }
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
        if (lane == 0 && e0 + e < E)
          s_logit[warp * MAX_EXPERTS + e0 + e] = acc[e] + (rb ? rb[e0 + e] : 0.f);
      }
    }
    __syncwarp();
    router_select(s_logit + warp * MAX_EXPERTS, lane, E, k, experts_out + static_cast<size_t>(t) * k,
                  gates_out + static_cast<size_t>(t) * k);
    __syncwarp();
    if constexpr (PREFETCH) {
#pragma unroll
      for (int it = 0; it < MAXIT; ++it) cur[it] = nxt[it];
    } else {
      if (t + stride < tokens) B200_LOAD_ROW(cur, t + stride);
    }
  }
#undef B200_LOAD_ROW
}

// One CTA per token: used for small token counts (decode), where a warp per
// token leaves most of the GPU idle.  The row stays in registers between the
// two passes (hidden <= 8192).
constexpr int RB_THREADS = 256;
constexpr int RB_MAXV = 4;  // 8-element vectors per thread

// Router for the token of this CTA.  Leaves the normalised row in `x` (this
// thread's 8-element vectors tid + v*RB_THREADS); writes it as fp16 to xn_row
// unless that is null; warp 0 writes the token's experts and gates.
template <typename T>
__device__ __forceinline__ void router_block_body(const T* __restrict__ row, int d, int E, int k,
                                                  float eps, const float* __restrict__ norm_w,
                                                  const float* __restrict__ rw,
                                                  const float* __restrict__ rb,
                                                  __half* __restrict__ xn_row,
                                                  int32_t* __restrict__ experts_row,
                                                  float* __restrict__ gates_row,
                                                  float (&x)[RB_MAXV][8]) {
  __shared__ float s_part[RB_THREADS / 32][8];
  __shared__ float s_logit[MAX_EXPERTS];
  __shared__ float s_ss[RB_THREADS / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nvec = d / 8;
  float ss = 0.f;
  float nw[RB_MAXV][8];  // norm weights: fetched with the row, not after the reduction (one memory latency less)
#pragma unroll
  for (int v = 0; v < RB_MAXV; ++v) {
    const int j = tid + v * RB_THREADS;
    if (j < nvec) {
      load8<T>(row + j * 8, x[v]);
      load8<float>(norm_w + j * 8, nw[v]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(x[v][i], x[v][i], ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) s_ss[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < RB_THREADS / 32; ++w) tot += s_ss[w];
  const float rstd = 1.0f / sqrtf(tot / static_cast<float>(d) + eps);
#pragma unroll
  for (int v = 0; v < RB_MAXV; ++v) {
    const int j = tid + v * RB_THREADS;
    if (j < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[v][i] = nw[v][i] * (x[v][i] * rstd);
      if (xn_row != nullptr) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          packed[i] = h2_as_u32(__halves2half2(to_half_sat(x[v][2 * i]), to_half_sat(x[v][2 * i + 1])));
        *reinterpret_cast<uint4*>(xn_row + j * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
  }
  for (int e0 = 0; e0 < E; e0 += 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int v = 0; v < RB_MAXV; ++v) {
      const int j = tid + v * RB_THREADS;
      if (j < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (e0 + e < E) {
            float r[8];
            load8<float>(rw + static_cast<size_t>(e0 + e) * d + j * 8, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[e] = fmaf(x[v][i], r[i], acc[e]);
          }
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
      if (lane == 0) s_part[warp][e] = acc[e];
    }
    __syncthreads();
    if (tid < 8 && e0 + tid < E) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < RB_THREADS / 32; ++w) v += s_part[w][tid];
      s_logit[e0 + tid] = v + (rb ? rb[e0 + tid] : 0.f);
    }
    __syncthreads();
  }
  if (warp == 0) router_select(s_logit, lane, E, k, experts_row, gates_row);
}

template <typename T>
__global__ void __launch_bounds__(RB_THREADS)
router_block_kernel(const T* __restrict__ h, int d, int E, int k, float eps,
                    const float* __restrict__ norm_w, const float* __restrict__ rw,
                    const float* __restrict__ rb, __half* __restrict__ xn_out,
                    int32_t* __restrict__ experts_out, float* __restrict__ gates_out) {
  const size_t t = blockIdx.x;
  float x[RB_MAXV][8];
  router_block_body<T>(h + t * d, d, E, k, eps, norm_w, rw, rb, xn_out + t * d,
                       experts_out + t * k, gates_out + t * k, x);
}

// ------------------------------------------------- fused decode front end
// Router, route plan and row permutation in one cooperative launch, one CTA
// per token (tokens <= FRONT_MAX_TOKENS).  After its token's experts are known
// every CTA meets the others at a grid-wide barrier, ranks its own k pairs
// among all pairs (stable by pair index, as route_plan_kernel does) and stores
// the normalised row, still in registers, at its k sorted positions.  Outputs
// are bit-identical to router_block_kernel + route_plan_kernel +
// permute_rows_kernel; the fp16 copy of the normalised rows is not written.
constexpr int FRONT_MAX_TOKENS = 128;
constexpr int FRONT_MAX_PAIRS = FRONT_MAX_TOKENS * MAX_TOPK;
constexpr int FRONT_PAIRS_PER_THREAD = FRONT_MAX_PAIRS / RB_THREADS;
constexpr int FRONT_SYNC_SLOTS = 32;

// {arrived, departed} per slot; zero between launches (the last CTA to leave
// the barrier resets its slot).  The host hands slots out in rotation, so up to
// FRONT_SYNC_SLOTS launches may be in flight on one device.
__device__ unsigned g_front_sync[FRONT_SYNC_SLOTS][2];

// Bounded grid-wide meeting point for a cooperative launch of `n` CTAs.
// Returns false if the others did not arrive within ~2^31 clock ticks (the
// status word then carries DEV_ERR_WAIT_TIMEOUT and the slot is left for the
// host to clear).
__device__ __forceinline__ bool front_grid_meet(unsigned* sync, unsigned n, int32_t* status) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&sync[0], 1u);
    const long long t0 = clock64();
    int ok = 1;
    while (*reinterpret_cast<volatile unsigned*>(&sync[0]) < n) {
      if (clock64() - t0 > (1ll << 31)) {
        atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        ok = 0;
        break;
      }
    }
    __threadfence();
    if (ok && atomicAdd(&sync[1], 1u) == n - 1) {
      // everyone has seen arrived == n: nobody reads the slot again
      *reinterpret_cast<volatile unsigned*>(&sync[0]) = 0;
      *reinterpret_cast<volatile unsigned*>(&sync[1]) = 0;
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

template <typename T>
__global__ void __launch_bounds__(RB_THREADS)
front_fused_kernel(const T* __restrict__ h, int d, int E, int k, float eps,
                   const float* __restrict__ norm_w, const float* __restrict__ rw,
                   const float* __restrict__ rb, int32_t* experts_out, float* __restrict__ gates_out,
                   int32_t* __restrict__ counts, int32_t* __restrict__ seg,
                   int32_t* __restrict__ perm, int32_t* __restrict__ inv, int kperm,
                   uint4* __restrict__ xs, unsigned* sync, int32_t* status) {
  __shared__ int s_total[MAX_EXPERTS];
  __shared__ int s_seg[MAX_EXPERTS + 1];
  __shared__ int s_rank[MAX_TOPK];
  const int tid = threadIdx.x;
  const int t = blockIdx.x, tokens = gridDim.x, pairs = tokens * k;
  float x[RB_MAXV][8];
  router_block_body<T>(h + static_cast<size_t>(t) * d, d, E, k, eps, norm_w, rw, rb, nullptr,
                       experts_out + static_cast<size_t>(t) * k, gates_out + static_cast<size_t>(t) * k, x);
  if (tid < MAX_EXPERTS) s_total[tid] = 0;
  if (tid < MAX_TOPK) s_rank[tid] = 0;
  if (!front_grid_meet(sync, static_cast<unsigned>(tokens), status)) return;

  // every CTA sees all pairs; mine are p0 .. p0+k-1
  const int p0 = t * k;
  int mine[MAX_TOPK];
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) mine[i] = i < k ? __ldcg(experts_out + p0 + i) : -1;
  int before[MAX_TOPK];
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) before[i] = 0;
#pragma unroll
  for (int r = 0; r < FRONT_PAIRS_PER_THREAD; ++r) {
    const int q = tid + r * RB_THREADS;
    if (q < pairs) {
      const int e = __ldcg(experts_out + q);
      if (e >= 0 && e < E) atomicAdd(&s_total[e], 1);
#pragma unroll
      for (int i = 0; i < MAX_TOPK; ++i)
        if (i < k && q < p0 + i && e == mine[i]) ++before[i];
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) {
    if (i < k) {
      int c = before[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
      if ((tid & 31) == 0 && c != 0) atomicAdd(&s_rank[i], c);
    }
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      s_seg[e] = run;
      run += s_total[e];
    }
    s_seg[E] = run;
  }
  __syncthreads();
  if (t == 0 && tid <= E) {
    seg[tid] = s_seg[tid];
    if (tid < E) counts[tid] = s_total[tid];
  }
  int pos[MAX_TOPK];
#pragma unroll
  for (int i = 0; i < MAX_TOPK; ++i) {
    pos[i] = i < k ? s_seg[mine[i]] + s_rank[i] : 0;
    if (i < k && tid == i) {
      perm[pos[i]] = p0 + i;
      inv[p0 + i] = pos[i];
    }
  }
  // the row goes from registers to its k sorted positions
  const int nvec = d / 8;
#pragma unroll
  for (int v = 0; v < RB_MAXV; ++v) {
    const int j = tid + v * RB_THREADS;
    if (j < nvec) {
      uint4 o;
      if (kperm) {  // halves in the order 0,4,1,5,2,6,3,7 (see permute_rows_kernel)
        o.x = h2_as_u32(__halves2half2(to_half_sat(x[v][0]), to_half_sat(x[v][4])));
        o.y = h2_as_u32(__halves2half2(to_half_sat(x[v][1]), to_half_sat(x[v][5])));
        o.z = h2_as_u32(__halves2half2(to_half_sat(x[v][2]), to_half_sat(x[v][6])));
        o.w = h2_as_u32(__halves2half2(to_half_sat(x[v][3]), to_half_sat(x[v][7])));
      } else {
        o.x = h2_as_u32(__halves2half2(to_half_sat(x[v][0]), to_half_sat(x[v][1])));
        o.y = h2_as_u32(__halves2half2(to_half_sat(x[v][2]), to_half_sat(x[v][3])));
        o.z = h2_as_u32(__halves2half2(to_half_sat(x[v][4]), to_half_sat(x[v][5])));
        o.w = h2_as_u32(__halves2half2(to_half_sat(x[v][6]), to_half_sat(x[v][7])));
      }
#pragma unroll
      for (int i = 0; i < MAX_TOPK; ++i) {
        if (i < k) xs[static_cast<size_t>(pos[i]) * nvec + j] = o;
      }
    }
  }
}

// Address of g_front_sync on the current device (cached per device).
static unsigned* front_sync_base() {
  static unsigned* ptrs[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
    set_error("front: no usable current device");
    return nullptr;
  }
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_front_sync);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaGetSymbolAddress(g_front_sync)");
      return nullptr;
    }
    ptrs[dev] = static_cast<unsigned*>(p);
  }
  return ptrs[dev];
}

bool front_fused_supported(int tokens, const b200moe_layer_t* L) {
  return tokens >= 1 && tokens <= FRONT_MAX_TOKENS && L->hidden <= 8 * RB_THREADS * RB_MAXV &&
         L->hidden % 256 == 0 && L->top_k >= 1 && L->top_k <= MAX_TOPK && L->experts <= MAX_EXPERTS;
}

int launch_front_fused(const void* h, int h_dtype, int tokens, const b200moe_layer_t* L,
                       int32_t* experts, float* gates, int32_t* counts, int32_t* seg,
                       int32_t* perm, int32_t* inv, int kperm, void* xs, int32_t* status,
                       cudaStream_t st) {
  B200_REQUIRE(front_fused_supported(tokens, L), "front: unsupported shape (tokens %d, hidden %d)",
               tokens, L->hidden);
  B200_REQUIRE(L->top_k <= L->experts, "front: top_k (%d) exceeds experts (%d)", L->top_k, L->experts);
  B200_REQUIRE(h_dtype == B200MOE_DT_F32 || h_dtype == B200MOE_DT_BF16,
               "front: activations must be fp32 or bf16");
  static std::atomic<unsigned> next_slot{0};
  unsigned* base = front_sync_base();
  if (base == nullptr) return B200MOE_ERR_CUDA;
  unsigned* sync = base + 2 * (next_slot.fetch_add(1) % FRONT_SYNC_SLOTS);
  int d = L->hidden, E = L->experts, k = L->top_k;
  float eps = L->rms_epsilon;
  const float* norm_w = L->ffn_norm_weight;
  const float* rw = L->router_weight;
  const float* rb = L->router_bias;
  uint4* xs4 = static_cast<uint4*>(xs);
  void* args[] = {&h, &d, &E, &k, &eps, &norm_w, &rw, &rb, &experts, &gates, &counts, &seg,
                  &perm, &inv, &kperm, &xs4, &sync, &status};
  const void* fn = h_dtype == B200MOE_DT_F32
                       ? reinterpret_cast<const void*>(&front_fused_kernel<float>)
                       : reinterpret_cast<const void*>(&front_fused_kernel<__nv_bfloat16>);
  // One CTA meets only itself at the grid barrier: an ordinary launch is enough
  // (and a few microseconds cheaper than a cooperative one) for a single token.
  if (tokens == 1)
    B200_CHECK_CUDA(cudaLaunchKernel(fn, dim3(1), dim3(RB_THREADS), args, 0, st));
  else
    B200_CHECK_CUDA(cudaLaunchCooperativeKernel(fn, dim3(tokens), dim3(RB_THREADS), args, 0, st));
  return B200MOE_OK;
}

int clear_front_sync(cudaStream_t st) {
  unsigned* base = front_sync_base();
  if (base == nullptr) return B200MOE_ERR_CUDA;
  B200_CHECK_CUDA(cudaMemsetAsync(base, 0, sizeof(unsigned) * 2 * FRONT_SYNC_SLOTS, st));
  return B200MOE_OK;
}

int launch_router(const void* h, int h_dtype, int tokens, const b200moe_layer_t* L, void* xn,
                  int32_t* experts, float* gates, cudaStream_t st) {
  B200_REQUIRE(L->hidden % 256 == 0, "router: hidden (%d) must be a multiple of 256", L->hidden);
  B200_REQUIRE(L->experts >= 1 && L->experts <= MAX_EXPERTS, "router: experts (%d) must be 1..64",
               L->experts);
  B200_REQUIRE(L->top_k >= 1 && L->top_k <= MAX_TOPK && L->top_k <= L->experts,
               "router: top_k (%d) must be 1..min(8, experts)", L->top_k);
  if (tokens == 0) return B200MOE_OK;
  B200_REQUIRE(h_dtype == B200MOE_DT_F32 || h_dtype == B200MOE_DT_BF16,
               "router: activations must be fp32 or bf16");
  if (tokens <= 512 && L->hidden <= 8 * RB_THREADS * RB_MAXV) {
    if (h_dtype == B200MOE_DT_F32)
      router_block_kernel<float><<<tokens, RB_THREADS, 0, st>>>(
          static_cast<const float*>(h), L->hidden, L->experts, L->top_k, L->rms_epsilon,
          L->ffn_norm_weight, L->router_weight, L->router_bias, static_cast<__half*>(xn), experts,
          gates);
    else
      router_block_kernel<__nv_bfloat16><<<tokens, RB_THREADS, 0, st>>>(
          static_cast<const __nv_bfloat16*>(h), L->hidden, L->experts, L->top_k, L->rms_epsilon,
          L->ffn_norm_weight, L->router_weight, L->router_bias, static_cast<__half*>(xn), experts,
          gates);
    B200_CHECK_CUDA(cudaGetLastError());
    return B200MOE_OK;
  }
  const size_t rs_smem = (static_cast<size_t>(L->experts) * L->hidden + L->hidden +
                          RS_WARPS * MAX_EXPERTS) * sizeof(float);
  if (tokens >= 1024 && rs_smem <= 227 * 1024) {
    const int ctas = min(sm_count(), (tokens + RS_WARPS - 1) / RS_WARPS);
    const void* fn;
    int which;
    if (h_dtype == B200MOE_DT_F32) {
      fn = reinterpret_cast<const void*>(&router_smem_kernel<float>); which = 0;
    } else if (L->hidden <= 4096) {
      fn = reinterpret_cast<const void*>(&router_smem_bf16_kernel<16, true>); which = 1;
    } else {  // longer rows do not fit the register file twice over: two passes over global memory
      fn = reinterpret_cast<const void*>(&router_smem_kernel<__nv_bfloat16>); which = 3;
    }
    static bool configured[16][4] = {};
    int dev = 0;
    B200_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 16 && !configured[dev][which]) {
      B200_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      configured[dev][which] = true;
    }
    int d_ = L->hidden, E_ = L->experts, k_ = L->top_k;
    float eps_ = L->rms_epsilon;
    const float *nw = L->ffn_norm_weight, *rwp = L->router_weight, *rbp = L->router_bias;
    __half* xnp = static_cast<__half*>(xn);
    void* args[] = {&h, &tokens, &d_, &E_, &k_, &eps_, &nw, &rwp, &rbp, &xnp, &experts, &gates};
    B200_CHECK_CUDA(cudaLaunchKernel(fn, dim3(ctas), dim3(RS_WARPS * 32), args, rs_smem, st));
    return B200MOE_OK;
  }
  dim3 grid((tokens + ROUTER_WARPS - 1) / ROUTER_WARPS), block(ROUTER_WARPS * 32);
  if (h_dtype == B200MOE_DT_F32) {
    router_kernel<float><<<grid, block, 0, st>>>(
        static_cast<const float*>(h), tokens, L->hidden, L->experts, L->top_k, L->rms_epsilon,
        L->ffn_norm_weight, L->router_weight, L->router_bias, static_cast<__half*>(xn), experts,
        gates);
  } else if (h_dtype == B200MOE_DT_BF16) {
    router_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(
        static_cast<const __nv_bfloat16*>(h), tokens, L->hidden, L->experts, L->top_k,
        L->rms_epsilon, L->ffn_norm_weight, L->router_weight, L->router_bias,
        static_cast<__half*>(xn), experts, gates);
  } else {
    B200_REQUIRE(false, "router: activations must be fp32 or bf16");
  }
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// -------------------------------------------------------------- route plan
// Stable counting sort of (token, slot) pairs by expert in one CTA: a shared
// histogram gives the segment offsets, then each 1024-pair chunk ranks its
// pairs with warp match/ballot masks and a per-expert scan over the 32 warps.
constexpr int PLAN_THREADS = 1024;

__global__ void __launch_bounds__(PLAN_THREADS)
route_plan_kernel(const int32_t* __restrict__ experts, int pairs, int e_begin, int E,
                  int32_t* __restrict__ counts, int32_t* __restrict__ seg,
                  int32_t* __restrict__ perm, int32_t* __restrict__ inv) {
  __shared__ int s_total[MAX_EXPERTS];
  __shared__ int s_run[MAX_EXPERTS];
  __shared__ int s_warp[32][MAX_EXPERTS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MAX_EXPERTS) s_total[tid] = 0;
  __syncthreads();
  for (int p = tid; p < pairs; p += PLAN_THREADS) {
    const int le = experts[p] - e_begin;
    if (le >= 0 && le < E) atomicAdd(&s_total[le], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      seg[e] = run;
      counts[e] = s_total[e];
      s_run[e] = run;
      run += s_total[e];
    }
    seg[E] = run;
  }
  __syncthreads();
  for (int base = 0; base < pairs; base += PLAN_THREADS) {
    const int p = base + tid;
    int le = -1;
    if (p < pairs) {
      le = experts[p] - e_begin;
      if (le < 0 || le >= E) le = -1;
    }
    for (int e = lane; e < E; e += 32) s_warp[warp][e] = 0;
    __syncwarp();
    const unsigned peers = __match_any_sync(0xffffffffu, le);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (le >= 0 && rank == 0) s_warp[warp][le] = __popc(peers);
    __syncthreads();
    if (tid < E) {
      int run = s_run[tid];
      for (int w = 0; w < 32; ++w) {
        const int c = s_warp[w][tid];
        s_warp[w][tid] = run;
        run += c;
      }
      s_run[tid] = run;
    }
    __syncthreads();
    if (p < pairs) {
      if (le >= 0) {
        const int pos = s_warp[warp][le] + rank;
        perm[pos] = p;
        inv[p] = pos;
      } else {
        inv[p] = -1;
      }
    }
    __syncthreads();
  }
}

int launch_route_plan(const int32_t* experts, int pairs, int e_begin, int E, int32_t* counts,
                      int32_t* seg, int32_t* perm, int32_t* inv, cudaStream_t st) {
  B200_REQUIRE(E >= 1 && E <= MAX_EXPERTS, "route_plan: local experts (%d) must be 1..64", E);
  B200_REQUIRE(pairs >= 0, "route_plan: negative pair count");
  route_plan_kernel<<<1, PLAN_THREADS, 0, st>>>(experts, pairs, e_begin, E, counts, seg, perm, inv);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// ------------------------------------------------------------ permute rows
// xs[pos,:] = xn[perm[pos]/k,:].  With kperm the eight halves of every 16-byte
// group are written in the order 0,4,1,5,2,6,3,7 — the order in which the Q4_K
// kernels pull nibble pairs out of a 32-bit word.
__global__ void __launch_bounds__(128)
permute_rows_kernel(const uint4* __restrict__ xn, const int32_t* __restrict__ perm,
                    const int32_t* __restrict__ seg, int E, int k, int vec_per_row, int kperm,
                    uint4* __restrict__ xs) {
  const int pos = blockIdx.x;
  if (pos >= seg[E]) return;
  const int tok = perm[pos] / k;
  const uint4* src = xn + static_cast<size_t>(tok) * vec_per_row;
  uint4* dst = xs + static_cast<size_t>(pos) * vec_per_row;
  for (int j = threadIdx.x; j < vec_per_row; j += blockDim.x) {
    uint4 v = src[j];
    if (kperm) {
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);  // (h0, h4)
      o.y = __byte_perm(v.x, v.z, 0x7632);  // (h1, h5)
      o.z = __byte_perm(v.y, v.w, 0x5410);  // (h2, h6)
      o.w = __byte_perm(v.y, v.w, 0x7632);  // (h3, h7)
      v = o;
    }
    dst[j] = v;
  }
}

int launch_permute_rows(const void* xn, const int32_t* perm, const int32_t* seg, int E, int pairs,
                        int k, int d, int kperm, void* xs, cudaStream_t st) {
  B200_REQUIRE(d % 8 == 0, "permute_rows: hidden must be a multiple of 8");
  if (pairs == 0) return B200MOE_OK;
  permute_rows_kernel<<<pairs, 128, 0, st>>>(static_cast<const uint4*>(xn), perm, seg, E, k,
                                             d / 8, kperm, static_cast<uint4*>(xs));
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// --------------------------------------------------- exchange plan (EP)
// Rows arrive from `world` source ranks, each rank's rows ordered by local
// expert: arrival order is (source, expert) blocks, the kernels want (expert,
// source) blocks.  counts[s*el + e] = rows from source s for local expert e.
// One CTA computes the segment offsets and both permutations.
__global__ void __launch_bounds__(1024)
exchange_plan_kernel(const int32_t* __restrict__ counts, int world, int el,
                     int32_t* __restrict__ seg, int32_t* __restrict__ perm,
                     int32_t* __restrict__ inv) {
  __shared__ int s_arr[MAX_EXPERTS * MAX_EXPERTS];  // arrival offset of block (s, e)
  __shared__ int s_srt[MAX_EXPERTS * MAX_EXPERTS];  // sorted offset of block (s, e)
  const int nb = world * el;
  if (threadIdx.x == 0) {
    int run = 0;
    for (int b = 0; b < nb; ++b) { s_arr[b] = run; run += counts[b]; }
    run = 0;
    for (int e = 0; e < el; ++e) {
      seg[e] = run;
      for (int s = 0; s < world; ++s) { s_srt[s * el + e] = run; run += counts[s * el + e]; }
    }
    seg[el] = run;
  }
  __syncthreads();
  for (int b = 0; b < nb; ++b) {
    const int c = counts[b], a0 = s_arr[b], p0 = s_srt[b];
    for (int i = threadIdx.x; i < c; i += blockDim.x) {
      perm[p0 + i] = a0 + i;
      inv[a0 + i] = p0 + i;
    }
  }
}

int launch_exchange_plan(const int32_t* counts, int world, int el, int32_t* seg, int32_t* perm,
                         int32_t* inv, cudaStream_t st) {
  B200_REQUIRE(world >= 1 && el >= 1 && world * el <= MAX_EXPERTS * MAX_EXPERTS && el <= MAX_EXPERTS,
               "exchange_plan: %d ranks x %d local experts out of range", world, el);
  exchange_plan_kernel<<<1, 1024, 0, st>>>(counts, world, el, seg, perm, inv);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// out[i,:] = rows[idx[i] / div,:] for i < n; rows of `vec_per_row` 16-byte vectors.
__global__ void __launch_bounds__(128)
gather_rows_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ idx, int div,
                   int vec_per_row, uint4* __restrict__ out) {
  const int i = blockIdx.x;
  const uint4* src = rows + static_cast<size_t>(idx[i] / div) * vec_per_row;
  uint4* dst = out + static_cast<size_t>(i) * vec_per_row;
  for (int j = threadIdx.x; j < vec_per_row; j += blockDim.x) dst[j] = src[j];
}

int launch_gather_rows(const void* rows, const int32_t* idx, int n, int div, int row_bytes,
                       void* out, cudaStream_t st) {
  B200_REQUIRE(row_bytes % 16 == 0 && div >= 1, "gather_rows: rows must be multiples of 16 bytes");
  if (n == 0) return B200MOE_OK;
  gather_rows_kernel<<<n, 128, 0, st>>>(static_cast<const uint4*>(rows), idx, div, row_bytes / 16,
                                        static_cast<uint4*>(out));
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// ----------------------------------------------------------------- combine
// One CTA per token: sum over slots (in slot order) of gate * (sum of the
// k-split partials of the pair's down-projection row), optional output RMS
// norm, residual add.
template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void store1(T* p, float v);
template <>
__device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

constexpr int COMBINE_THREADS = 256;

// four consecutive elements at once (16-byte / 8-byte accesses)
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(raw.x << 16);
  v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16);
  v[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
  const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// gate-weighted sum over the token's slots for four columns; per element the
// same operations in the same order as a scalar loop over slots and partials
template <typename TD>
__device__ __forceinline__ void combine4(const TD* __restrict__ dpart, int ksplit, size_t part_stride,
                                         const int (&pos)[MAX_TOPK], const float (&gate)[MAX_TOPK],
                                         int k, int d, int j, float (&acc)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = 0.f;
#pragma unroll
  for (int s = 0; s < MAX_TOPK; ++s) {
    if (s < k && pos[s] >= 0) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < ksplit; ++c) {
        float p4[4];
        load4<TD>(dpart + c * part_stride + static_cast<size_t>(pos[s]) * d + j, p4);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += p4[i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] += gate[s] * v[i];
    }
  }
}

template <typename TD, typename TH, typename TY>
__global__ void __launch_bounds__(COMBINE_THREADS)
combine_kernel(const TD* __restrict__ dpart, int ksplit, size_t part_stride,
               const int32_t* __restrict__ inv, const float* __restrict__ gates,
               const TH* __restrict__ h, int d, int k, const float* __restrict__ out_norm_w,
               float eps, int add_residual, TY* __restrict__ y) {
  extern __shared__ float s_row[];
  __shared__ float s_red[COMBINE_THREADS / 32];
  const size_t t = blockIdx.x;
  int pos[MAX_TOPK];
  float gate[MAX_TOPK];
#pragma unroll
  for (int s = 0; s < MAX_TOPK; ++s) {
    pos[s] = s < k ? inv[t * k + s] : -1;
    gate[s] = s < k ? gates[t * k + s] : 0.f;
  }
  if (gridDim.y > 1) {
    // no output norm: column slices are independent, one slice per blockIdx.y
    const int per = ((d / 4 + gridDim.y - 1) / gridDim.y) * 4;
    const int j0 = blockIdx.y * per, j1 = min(d, j0 + per);
    for (int j = j0 + threadIdx.x * 4; j < j1; j += COMBINE_THREADS * 4) {
      float acc[4];
      combine4<TD>(dpart, ksplit, part_stride, pos, gate, k, d, j, acc);
      if (add_residual) {
        float r[4];
        load4<TH>(h + t * d + j, r);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += r[i];
      }
      store4<TY>(y + t * d + j, acc);
    }
    return;
  }
  float ss = 0.f;
  for (int j = threadIdx.x * 4; j < d; j += COMBINE_THREADS * 4) {
    float acc[4];
    combine4<TD>(dpart, ksplit, part_stride, pos, gate, k, d, j, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s_row[j + i] = acc[i];
      ss = fmaf(acc[i], acc[i], ss);
    }
  }
  float scale = 1.f;
  if (out_norm_w != nullptr && add_residual) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < COMBINE_THREADS / 32; ++w) tot += s_red[w];
    scale = 1.0f / sqrtf(tot / static_cast<float>(d) + eps);
  }
  // every thread re-reads only the columns it wrote itself
  for (int j = threadIdx.x * 4; j < d; j += COMBINE_THREADS * 4) {
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = s_row[j + i];
    if (add_residual) {
      float r[4];
      load4<TH>(h + t * d + j, r);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (out_norm_w != nullptr) v[i] = out_norm_w[j + i] * (v[i] * scale);
        v[i] += r[i];
      }
    }
    store4<TY>(y + t * d + j, v);
  }
}

int launch_combine(const void* dpart, int d_dtype, int ksplit, int pairs, const int32_t* inv,
                   const float* gates, const void* h, int h_dtype, int tokens,
                   const b200moe_layer_t* L, int add_residual, void* y, int y_dtype,
                   cudaStream_t st) {
  if (tokens == 0) return B200MOE_OK;
  const int d = L->hidden, k = L->top_k;
  const size_t smem = static_cast<size_t>(d) * sizeof(float);
  B200_REQUIRE(smem <= 48 * 1024, "combine: hidden (%d) too large", d);
  B200_REQUIRE(d % 4 == 0 && k >= 1 && k <= MAX_TOPK, "combine: hidden must be a multiple of 4, top_k 1..8");
  const size_t stride = static_cast<size_t>(pairs) * d;
  const bool need_row = L->layer_output_norm_weight != nullptr && add_residual;
  int slices = 1;
  if (!need_row && tokens < 1024) slices = max(1, min(d / COMBINE_THREADS, 2048 / tokens));
  dim3 grid(tokens, slices), block(COMBINE_THREADS);
#define LAUNCH(TD, TH, TY)                                                                     \
  combine_kernel<TD, TH, TY><<<grid, block, smem, st>>>(static_cast<const TD*>(dpart), ksplit,   \
                                                        stride, inv, gates,                      \
                                                        static_cast<const TH*>(h), d, k,         \
                                                        L->layer_output_norm_weight,             \
                                                        L->rms_epsilon, add_residual,            \
                                                        static_cast<TY*>(y))
  const bool dbf = d_dtype == B200MOE_DT_BF16;
  B200_REQUIRE(dbf || d_dtype == B200MOE_DT_F32, "combine: partial rows must be fp32 or bf16");
  if (h_dtype == B200MOE_DT_F32 && y_dtype == B200MOE_DT_F32) {
    if (dbf) LAUNCH(__nv_bfloat16, float, float); else LAUNCH(float, float, float);
  } else if (h_dtype == B200MOE_DT_BF16 && y_dtype == B200MOE_DT_BF16) {
    if (dbf) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16); else LAUNCH(float, __nv_bfloat16, __nv_bfloat16);
  } else if (h_dtype == B200MOE_DT_BF16 && y_dtype == B200MOE_DT_F32) {
    if (dbf) LAUNCH(__nv_bfloat16, __nv_bfloat16, float); else LAUNCH(float, __nv_bfloat16, float);
  } else {
    B200_REQUIRE(false, "combine: unsupported dtype pair (%d, %d)", h_dtype, y_dtype);
  }
#undef LAUNCH
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// ----------------------------------------------------- reference dequantise
template <typename TO>
__global__ void dequant_q8_kernel(const int8_t* __restrict__ qs, const __half* __restrict__ d,
                                  size_t n, TO* __restrict__ out) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const __half scale = d[i >> 5];
  if constexpr (sizeof(TO) == 2) {
    out[i] = __hmul(scale, __int2half_rn(qs[i]));
  } else {
    out[i] = __half2float(scale) * static_cast<float>(qs[i]);
  }
}

template <typename TO>
__global__ void dequant_q4k_kernel(const uint8_t* __restrict__ qs, const __half2* __restrict__ sub,
                                   size_t n, TO* __restrict__ out) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const uint8_t b = qs[i >> 1];
  const int q = (i & 1) ? (b >> 4) : (b & 0xF);
  const __half2 sm = sub[i >> 5];
  // the _rn forms are never contracted into an fma: the reference rounds after
  // the product and again after the subtraction
  const __half w = __hsub_rn(__hmul_rn(__low2half(sm), __int2half_rn(q)), __high2half(sm));
  if constexpr (sizeof(TO) == 2) {
    out[i] = w;
  } else {
    out[i] = __half2float(w);
  }
}

template <typename TO>
__global__ void dequant_f16_kernel(const __half* __restrict__ w, size_t n, TO* __restrict__ out) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  if constexpr (sizeof(TO) == 2) {
    out[i] = w[i];
  } else {
    out[i] = __half2float(w[i]);
  }
}

int launch_dequant(const b200moe_weight_t* w, int out_dtype, void* out, cudaStream_t st) {
  B200_REQUIRE(out_dtype == B200MOE_DT_F16 || out_dtype == B200MOE_DT_F32,
               "dequant: out_dtype must be fp16 or fp32");
  const size_t n = static_cast<size_t>(w->experts) * w->rows * w->cols;
  if (n == 0) return B200MOE_OK;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  const bool f16 = out_dtype == B200MOE_DT_F16;
  switch (w->layout) {
    case B200MOE_LAYOUT_Q8_0:
      B200_REQUIRE(w->cols % 32 == 0, "dequant: Q8_0 needs cols %% 32 == 0");
      if (f16)
        dequant_q8_kernel<__half><<<blocks, threads, 0, st>>>(
            static_cast<const int8_t*>(w->qs), static_cast<const __half*>(w->d), n,
            static_cast<__half*>(out));
      else
        dequant_q8_kernel<float><<<blocks, threads, 0, st>>>(
            static_cast<const int8_t*>(w->qs), static_cast<const __half*>(w->d), n,
            static_cast<float*>(out));
      break;
    case B200MOE_LAYOUT_Q4_K:
      B200_REQUIRE(w->cols % 256 == 0, "dequant: Q4_K needs cols %% 256 == 0");
      if (f16)
        dequant_q4k_kernel<__half><<<blocks, threads, 0, st>>>(
            static_cast<const uint8_t*>(w->qs), static_cast<const __half2*>(w->sub), n,
            static_cast<__half*>(out));
      else
        dequant_q4k_kernel<float><<<blocks, threads, 0, st>>>(
            static_cast<const uint8_t*>(w->qs), static_cast<const __half2*>(w->sub), n,
            static_cast<float*>(out));
      break;
    case B200MOE_LAYOUT_F16:
      if (f16)
        dequant_f16_kernel<__half><<<blocks, threads, 0, st>>>(static_cast<const __half*>(w->qs),
                                                               n, static_cast<__half*>(out));
      else
        dequant_f16_kernel<float><<<blocks, threads, 0, st>>>(static_cast<const __half*>(w->qs),
                                                              n, static_cast<float*>(out));
      break;
    default:
      B200_REQUIRE(false, "dequant: unknown layout %d", w->layout);
  }
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// ------------------------------------------------- Q8_0 scale transposition
// d [rows, K/32] -> [K/256][rows][8]: the eight scales one row needs for a
// 256-k stage become 16 contiguous bytes and consecutive rows are adjacent, so
// a stage's scale tile is one contiguous run (one bulk copy instead of one
// 16-byte TMA request per row).
__global__ void q8_scales_tile_kernel(const uint4* __restrict__ d, long long rows, int groups,
                                      uint4* __restrict__ out) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= rows * groups) return;
  const long long r = i / groups;
  const int g = static_cast<int>(i % groups);
  out[static_cast<long long>(g) * rows + r] = d[i];
}

int launch_q8_prepare(const void* d, long long rows, int cols, void* out, cudaStream_t st) {
  B200_REQUIRE(cols % 256 == 0, "q8_prepare: cols (%d) must be a multiple of 256", cols);
  const int groups = cols / 256;
  const long long n = rows * groups;
  if (n == 0) return B200MOE_OK;
  q8_scales_tile_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const uint4*>(d), rows, groups, static_cast<uint4*>(out));
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// --------------------------------------------------------- Q4_K scale fold
// One thread per super-block: the eight 6-bit sub-scales / sub-mins
// (low nibble plane | 2-bit high plane << 4) times d / dmin, each product
// rounded once to fp16.
__global__ void q4k_prepare_kernel(const __half* __restrict__ d, const __half* __restrict__ dmin,
                                   const uint8_t* __restrict__ sh, const uint8_t* __restrict__ sl,
                                   const uint8_t* __restrict__ mh, const uint8_t* __restrict__ ml,
                                   long long blocks, __half2* __restrict__ sub) {
  const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (b >= blocks) return;
  const __half dd = d[b], dm = dmin[b];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int sc = ((sl[b * 4 + (i >> 1)] >> ((i & 1) * 4)) & 0xF) |
                   (((sh[b * 2 + (i >> 2)] >> ((i & 3) * 2)) & 3) << 4);
    const int mn = ((ml[b * 4 + (i >> 1)] >> ((i & 1) * 4)) & 0xF) |
                   (((mh[b * 2 + (i >> 2)] >> ((i & 3) * 2)) & 3) << 4);
    sub[b * 8 + i] = __halves2half2(__hmul(dd, __int2half_rn(sc)), __hmul(dm, __int2half_rn(mn)));
  }
}

int launch_q4k_prepare(const void* d, const void* dmin, const uint8_t* sh, const uint8_t* sl,
                       const uint8_t* mh, const uint8_t* ml, long long blocks, void* sub,
                       cudaStream_t st) {
  if (blocks == 0) return B200MOE_OK;
  const int threads = 256;
  q4k_prepare_kernel<<<static_cast<unsigned>((blocks + threads - 1) / threads), threads, 0, st>>>(
      static_cast<const __half*>(d), static_cast<const __half*>(dmin), sh, sl, mh, ml, blocks,
      static_cast<__half2*>(sub));
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// ------------------------------------------------------------- GGUF unpack
// Q8_0 file block: fp16 scale + 32 int8.  One thread per quant.
__global__ void gguf_q8_kernel(const uint8_t* __restrict__ raw, long long blocks,
                               uint16_t* __restrict__ d, int8_t* __restrict__ qs) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= blocks * 32) return;
  const long long b = i >> 5;
  const int j = static_cast<int>(i & 31);
  const uint8_t* blk = raw + b * 34;
  qs[i] = static_cast<int8_t>(blk[2 + j]);
  if (j == 0) d[b] = static_cast<uint16_t>(blk[0]) | (static_cast<uint16_t>(blk[1]) << 8);
}

// Q4_K file super-block (144 B): d, dmin, 12 bytes of 6-bit fields, 128 bytes
// of nibbles.  One thread per super-block writes the planar planes.
__global__ void gguf_q4k_kernel(const uint8_t* __restrict__ raw, long long blocks,
                                uint16_t* __restrict__ d, uint16_t* __restrict__ dmin,
                                uint8_t* __restrict__ sh, uint8_t* __restrict__ sl,
                                uint8_t* __restrict__ mh, uint8_t* __restrict__ ml,
                                uint8_t* __restrict__ qs) {
  const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (b >= blocks) return;
  const uint8_t* blk = raw + b * 144;
  d[b] = static_cast<uint16_t>(blk[0]) | (static_cast<uint16_t>(blk[1]) << 8);
  dmin[b] = static_cast<uint16_t>(blk[2]) | (static_cast<uint16_t>(blk[3]) << 8);
  const uint8_t* s = blk + 4;
  uint8_t sc[8], mn[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    sc[i] = s[i] & 63;
    mn[i] = s[i + 4] & 63;
    sc[i + 4] = (s[i + 8] & 0xF) | ((s[i] >> 6) << 4);
    mn[i + 4] = (s[i + 8] >> 4) | ((s[i + 4] >> 6) << 4);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    sl[b * 4 + j] = (sc[2 * j] & 0xF) | ((sc[2 * j + 1] & 0xF) << 4);
    ml[b * 4 + j] = (mn[2 * j] & 0xF) | ((mn[2 * j + 1] & 0xF) << 4);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    sh[b * 2 + j] = (sc[4 * j] >> 4) | ((sc[4 * j + 1] >> 4) << 2) | ((sc[4 * j + 2] >> 4) << 4) |
                    ((sc[4 * j + 3] >> 4) << 6);
    mh[b * 2 + j] = (mn[4 * j] >> 4) | ((mn[4 * j + 1] >> 4) << 2) | ((mn[4 * j + 2] >> 4) << 4) |
                    ((mn[4 * j + 3] >> 4) << 6);
  }
  const uint8_t* q = blk + 16;
  uint8_t* o = qs + b * 128;
  for (int g = 0; g < 4; ++g) {
    for (int i = 0; i < 16; ++i) {
      const uint8_t a = q[32 * g + 2 * i], c = q[32 * g + 2 * i + 1];
      o[(2 * g) * 16 + i] = (a & 0xF) | ((c & 0xF) << 4);
      o[(2 * g + 1) * 16 + i] = (a >> 4) | ((c >> 4) << 4);
    }
  }
}

int launch_gguf_q8(const uint8_t* raw, long long blocks, void* d, int8_t* qs, cudaStream_t st) {
  if (blocks == 0) return B200MOE_OK;
  const long long n = blocks * 32;
  gguf_q8_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      raw, blocks, static_cast<uint16_t*>(d), qs);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

int launch_gguf_q4k(const uint8_t* raw, long long blocks, void* d, void* dmin, uint8_t* sh,
                    uint8_t* sl, uint8_t* mh, uint8_t* ml, uint8_t* qs, cudaStream_t st) {
  if (blocks == 0) return B200MOE_OK;
  gguf_q4k_kernel<<<static_cast<unsigned>((blocks + 127) / 128), 128, 0, st>>>(
      raw, blocks, static_cast<uint16_t*>(d), static_cast<uint16_t*>(dmin), sh, sl, mh, ml, qs);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

}  // namespace b200moe
