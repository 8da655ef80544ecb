// The attention block that precedes every MoE layer: RMS norm, rotary embedding
// fused with the paged KV-cache write, and decode attention that reads K and V
// straight from the cache pages through the page table (no linearised copy).
//
// Page slab layout (one row per page):
//   [transformer block][K | V][position in page][kv head][head dim]
// i.e. the K (or V) row of one position and kv head is head_dim contiguous
// elements, and consecutive positions of a page are kv_heads*head_dim apart.
#include "kernels.h"

namespace b200moe {
namespace {

__device__ __forceinline__ float ld_elem(const void* p, int dtype, size_t i) {
  if (dtype == B200MOE_DT_F32) return static_cast<const float*>(p)[i];
  if (dtype == B200MOE_DT_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_elem(void* p, int dtype, size_t i, float v) {
  if (dtype == B200MOE_DT_F32) static_cast<float*>(p)[i] = v;
  else if (dtype == B200MOE_DT_F16) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
inline size_t dt_bytes(int dt) { return dt == B200MOE_DT_F32 ? 4 : 2; }

// ------------------------------------------------------------------ RMS norm
// y = w * (x * rsqrt(mean(x^2) + eps)), fp32 arithmetic, one CTA per row.
__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const void* __restrict__ x, int x_dtype, const float* __restrict__ w, int d, float eps,
                     void* __restrict__ y, int y_dtype) {
  __shared__ float s_red[8];
  const size_t row = blockIdx.x;
  float ss = 0.f;
  for (int j = threadIdx.x; j < d; j += 256) {
    const float v = ld_elem(x, x_dtype, row * d + j);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_red[i];
  const float rstd = 1.0f / sqrtf(tot / static_cast<float>(d) + eps);
  for (int j = threadIdx.x; j < d; j += 256)
    st_elem(y, y_dtype, row * d + j, w[j] * (ld_elem(x, x_dtype, row * d + j) * rstd));
}

// ------------------------------------------- rotary embedding + KV page write
// One CTA per token.  q is rotated in place; k is rotated and, with v, written
// to its slot of the page the token's position falls in (and, for prefill, to
// contiguous k_out / v_out so that the attention over the fresh K/V needs no
// read-back).  Pairs (2i, 2i+1) share the angle position * freq[i].
struct RopeArgs {
  void* q;            // [tokens, heads, hd] in/out
  const void* k;      // [tokens, kv_heads, hd]
  const void* v;
  void* k_out;        // NULL or [tokens, kv_heads, hd]
  void* v_out;
  int io_dtype;
  void* slab;
  int cache_dtype;
  const int32_t* positions;  // [tokens] absolute position of every token
  const int32_t* page_ids;   // [bs, pages_per_seq]
  const float* freqs;        // [hd / 2]
  int tokens, tokens_per_seq, pages_per_seq, page_count;
  int heads, kv_heads, hd, stride, blocks, block_index;
  int32_t* status;
};

__global__ void __launch_bounds__(128) rope_kv_write_kernel(const RopeArgs a) {
  const int t = blockIdx.x;
  const int b = t / a.tokens_per_seq;
  const int pos = a.positions[t];
  const int hpairs = a.hd / 2;
  const int page_slot = pos / a.stride;
  long long page = -1;
  if (pos >= 0 && page_slot < a.pages_per_seq) page = a.page_ids[b * a.pages_per_seq + page_slot];
  if (page < 0 || page >= a.page_count) {
    if (threadIdx.x == 0) atomicOr(a.status, DEV_ERR_BOUNDS);
    page = -1;  // rotate q, skip the cache write
  }
  const float fpos = static_cast<float>(pos);
  // q heads
  for (int i = threadIdx.x; i < a.heads * hpairs; i += 128) {
    const int hh = i / hpairs, j = i % hpairs;
    float sn, cs;
    sincosf(fpos * a.freqs[j], &sn, &cs);
    const size_t base = (static_cast<size_t>(t) * a.heads + hh) * a.hd + 2 * j;
    const float re = ld_elem(a.q, a.io_dtype, base), im = ld_elem(a.q, a.io_dtype, base + 1);
    st_elem(a.q, a.io_dtype, base, re * cs - im * sn);
    st_elem(a.q, a.io_dtype, base + 1, im * cs + re * sn);
  }
  // k (rotated) and v heads
  const size_t row_elems = static_cast<size_t>(a.kv_heads) * a.hd;
  const size_t page_elems = static_cast<size_t>(a.blocks) * 2 * a.stride * row_elems;
  const size_t k_slot = page < 0 ? 0
                                 : static_cast<size_t>(page) * page_elems +
                                       ((static_cast<size_t>(a.block_index) * 2 + 0) * a.stride + pos % a.stride) * row_elems;
  const size_t v_slot = k_slot + static_cast<size_t>(a.stride) * row_elems;
  for (int i = threadIdx.x; i < a.kv_heads * hpairs; i += 128) {
    const int hh = i / hpairs, j = i % hpairs;
    float sn, cs;
    sincosf(fpos * a.freqs[j], &sn, &cs);
    const size_t src = (static_cast<size_t>(t) * a.kv_heads + hh) * a.hd + 2 * j;
    const float re = ld_elem(a.k, a.io_dtype, src), im = ld_elem(a.k, a.io_dtype, src + 1);
    // rounded to the activation dtype first, as the reference's rotated K is
    const float kr = re * cs - im * sn, ki = im * cs + re * sn;
    const float v0 = ld_elem(a.v, a.io_dtype, src), v1 = ld_elem(a.v, a.io_dtype, src + 1);
    if (a.k_out != nullptr) {
      st_elem(a.k_out, a.io_dtype, src, kr);
      st_elem(a.k_out, a.io_dtype, src + 1, ki);
      st_elem(a.v_out, a.io_dtype, src, v0);
      st_elem(a.v_out, a.io_dtype, src + 1, v1);
    }
    if (page >= 0) {
      const size_t dst = static_cast<size_t>(hh) * a.hd + 2 * j;
      float kr_c = kr, ki_c = ki;
      if (a.io_dtype == B200MOE_DT_BF16) {
        kr_c = __bfloat162float(__float2bfloat16_rn(kr));
        ki_c = __bfloat162float(__float2bfloat16_rn(ki));
      } else if (a.io_dtype == B200MOE_DT_F16) {
        kr_c = __half2float(__float2half_rn(kr));
        ki_c = __half2float(__float2half_rn(ki));
      }
      st_elem(a.slab, a.cache_dtype, k_slot + dst, kr_c);
      st_elem(a.slab, a.cache_dtype, k_slot + dst + 1, ki_c);
      st_elem(a.slab, a.cache_dtype, v_slot + dst, v0);
      st_elem(a.slab, a.cache_dtype, v_slot + dst + 1, v1);
    }
  }
}

// ------------------------------------------------------- paged decode attention
// One CTA per (position split, kv head, sequence): the G = heads / kv_heads query
// heads that share the kv head are processed together, so every K and V row is
// read once per split.  Per step of 128 positions:
//   1. the K rows and the V rows of the step are copied into shared memory with
//      cp.async (16 bytes per lane, a row's bytes by consecutive lanes: fully
//      coalesced; V's copy stays in flight during 2 and 3);
//   2. thread t scores position t for all G heads from its shared-memory row
//      (rows are padded by 16 bytes so that 16-byte row reads of a quarter warp
//      hit all 32 banks);
//   3. block-wide online-softmax update;
//   4. thread t accumulates output column d = t % hd over the step's positions
//      from the V tile.
// Splits are merged by a second kernel.
constexpr int AD_THREADS = 128;
constexpr int AD_MAXG = 8;

template <typename TC>
struct CacheVec;  // 16-byte vector of cache elements -> floats
template <>
struct CacheVec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  }
  __device__ static float one(const float* p) { return *p; }
};
template <>
struct CacheVec<__half> {
  static constexpr int N = 8;
  __device__ static void load(const __half* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(u32_as_h2(w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static float one(const __half* p) { return __half2float(*p); }
};
template <>
struct CacheVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static float one(const __nv_bfloat16* p) { return __bfloat162float(*p); }
};

struct DecodeArgs {
  const void* q;      // [bs, heads, hd] rotated
  int q_dtype;
  const void* slab;
  const int32_t* page_ids;  // [bs, pages_per_seq]
  const int32_t* seq_lens;  // [bs] positions to attend (the new one included)
  float* partial;     // [bs, kv_heads, splits, G, hd + 2]
  int bs, heads, kv_heads, hd, stride, blocks, block_index, pages_per_seq, page_count, splits;
  float scale, softcap;  // softcap <= 0: none
  int32_t* status;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename TC, int HD>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(const DecodeArgs a) {
  constexpr int GROUPS = AD_THREADS / HD;        // position groups in the P.V phase (hd 128: 1, hd 64: 2)
  constexpr int ROW_B = HD * sizeof(TC);         // bytes of one K or V row
  constexpr int ROW_PAD = ROW_B + 16;            // shared-memory row pitch
  constexpr int CHUNKS = ROW_B / 16;             // 16-byte pieces per row
  extern __shared__ __align__(16) uint8_t s_tiles[];  // K tile, then V tile: 2 x 128 x ROW_PAD
  __shared__ float s_q[AD_MAXG][HD];
  __shared__ float s_p[AD_MAXG][AD_THREADS];
  __shared__ long long s_row[AD_THREADS];        // element offset of each position's K row, -1 = none
  __shared__ float s_red[AD_MAXG][AD_THREADS / 32];
  __shared__ float s_m[AD_MAXG], s_l[AD_MAXG], s_alpha[AD_MAXG];
  uint8_t* s_k = s_tiles;
  uint8_t* s_v = s_tiles + AD_THREADS * ROW_PAD;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int G = a.heads / a.kv_heads;
  const int seq_len = a.seq_lens[b];
  const TC* slab = static_cast<const TC*>(a.slab);
  const size_t row_elems = static_cast<size_t>(a.kv_heads) * HD;
  const size_t page_elems = static_cast<size_t>(a.blocks) * 2 * a.stride * row_elems;
  const size_t v_off = static_cast<size_t>(a.stride) * row_elems;  // V row = K row + this many elements

  for (int i = t; i < G * HD; i += AD_THREADS) {
    const int g = i / HD, d = i % HD;
    s_q[g][d] = ld_elem(a.q, a.q_dtype, (static_cast<size_t>(b) * a.heads + kvh * G + g) * HD + d) * a.scale;
  }
  if (t < AD_MAXG) { s_m[t] = -INFINITY; s_l[t] = 0.f; }

  // positions of this split, in whole steps of 128
  const int steps_total = (seq_len + AD_THREADS - 1) / AD_THREADS;
  const int steps_per = (steps_total + a.splits - 1) / a.splits;
  const int p_begin = split * steps_per * AD_THREADS;
  const int p_end = min(seq_len, (split + 1) * steps_per * AD_THREADS);

  const int d_own = t % HD, grp = t / HD;
  float acc[AD_MAXG];
#pragma unroll
  for (int g = 0; g < AD_MAXG; ++g) acc[g] = 0.f;

  for (int p0 = p_begin; p0 < p_end; p0 += AD_THREADS) {
    const int n_here = min(AD_THREADS, p_end - p0);
    // row offsets of the step's positions
    {
      const int pos = p0 + t;
      long long row = -1;
      if (t < n_here) {
        const int slot = pos / a.stride;
        const long long page = slot < a.pages_per_seq ? a.page_ids[b * a.pages_per_seq + slot] : -1;
        if (page < 0 || page >= a.page_count) {
          atomicOr(a.status, DEV_ERR_BOUNDS);
        } else {
          row = static_cast<long long>(static_cast<size_t>(page) * page_elems +
                                       ((static_cast<size_t>(a.block_index) * 2) * a.stride + pos % a.stride) * row_elems +
                                       static_cast<size_t>(kvh) * HD);
        }
      }
      s_row[t] = row;
    }
    __syncthreads();
    // K tile, then V tile, 16 bytes per lane per copy
    for (int i = t; i < n_here * CHUNKS; i += AD_THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const long long row = s_row[r];
      if (row >= 0) cp_async16(smem_u32(s_k + r * ROW_PAD + c * 16), slab + row + c * (16 / sizeof(TC)));
    }
    cp_async_commit();
    for (int i = t; i < n_here * CHUNKS; i += AD_THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const long long row = s_row[r];
      if (row >= 0) cp_async16(smem_u32(s_v + r * ROW_PAD + c * 16), slab + row + v_off + c * (16 / sizeof(TC)));
    }
    cp_async_commit();
    cp_async_wait<1>();  // K has landed (this thread's copies)
    __syncthreads();     // everyone's
    float sc[AD_MAXG];
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) sc[g] = -INFINITY;
    if (t < n_here && s_row[t] >= 0) {
      float dot[AD_MAXG];
#pragma unroll
      for (int g = 0; g < AD_MAXG; ++g) dot[g] = 0.f;
      constexpr int N = CacheVec<TC>::N;
      const TC* krow = reinterpret_cast<const TC*>(s_k + t * ROW_PAD);
#pragma unroll 4
      for (int c = 0; c < HD / N; ++c) {
        float kv[N];
        CacheVec<TC>::load(krow + c * N, kv);
#pragma unroll
        for (int g = 0; g < AD_MAXG; ++g) {
          if (g < G) {
#pragma unroll
            for (int i = 0; i < N; ++i) dot[g] = fmaf(kv[i], s_q[g][c * N + i], dot[g]);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < AD_MAXG; ++g) {
        if (g < G) sc[g] = a.softcap > 0.f ? a.softcap * tanhf(dot[g] / a.softcap) : dot[g];
      }
    }
    // block maximum per head
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) {
      if (g < G) {
        float m = sc[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) s_red[g][warp] = m;
      }
    }
    __syncthreads();
    if (t < G) {
      float m = s_m[t];
      for (int w = 0; w < AD_THREADS / 32; ++w) m = fmaxf(m, s_red[t][w]);
      s_alpha[t] = (m == -INFINITY) ? 1.f : __expf(s_m[t] - m);  // exp(-inf) = 0 on the first step
      s_m[t] = m;
    }
    __syncthreads();
    // probabilities and their block sum
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) {
      if (g < G) {
        const float p = (sc[g] == -INFINITY) ? 0.f : __expf(sc[g] - s_m[g]);
        s_p[g][t] = p;
        float s = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) s_red[g][warp] = s;
      }
    }
    cp_async_wait<0>();  // V has landed
    __syncthreads();
    if (t < G) {
      float s = 0.f;
      for (int w = 0; w < AD_THREADS / 32; ++w) s += s_red[t][w];
      s_l[t] = s_l[t] * s_alpha[t] + s;
    }
    // P.V: thread owns column d_own for the positions j = grp, grp + GROUPS, ...
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g)
      if (g < G) acc[g] *= s_alpha[g];
    for (int j = grp; j < n_here; j += GROUPS) {
      if (s_row[j] < 0) continue;
      const float v = CacheVec<TC>::one(reinterpret_cast<const TC*>(s_v + j * ROW_PAD) + d_own);
#pragma unroll
      for (int g = 0; g < AD_MAXG; ++g)
        if (g < G) acc[g] = fmaf(s_p[g][j], v, acc[g]);
    }
    __syncthreads();  // s_row, s_p and the tiles are rewritten by the next step
  }

  // merge the position groups, write this split's partial (unnormalised sums, max, denominator)
  float* out = a.partial + ((static_cast<size_t>(b) * a.kv_heads + kvh) * a.splits + split) * G * (HD + 2);
  // (loops over g are unrolled with a static bound: a dynamically indexed acc[]
  // would live in local memory for the whole kernel)
  if constexpr (GROUPS > 1) {
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) {
      if (g < G) {
        __syncthreads();
        s_p[0][t] = acc[g];
        __syncthreads();
        if (grp == 0) {
          float s = 0.f;
          for (int q = 0; q < GROUPS; ++q) s += s_p[0][q * HD + d_own];
          out[g * (HD + 2) + d_own] = s;
        }
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g)
      if (g < G) out[g * (HD + 2) + d_own] = acc[g];
  }
  if (t < G) {
    out[t * (HD + 2) + HD] = s_m[t];
    out[t * (HD + 2) + HD + 1] = s_l[t];
  }
}

// ---- the same on tensor cores, for 16-bit caches -----------------------------
// Scores and outputs as mma.sync.m16n8k16 products with the G query heads as the
// M dimension (padded to 16):  S[head][pos] = Q[head][:] . K[pos][:]  and
// O[head][d] = sum_pos P[head][pos] V[pos][d].  The accumulator fragment of S is,
// element for element, the A fragment of P for the second product, so the
// probabilities never leave registers.  Four warps per CTA; per stage of 64
// positions every warp owns 16 of them with its own online-softmax state; the K
// and V rows of a stage arrive by cp.async (16 bytes per lane, coalesced, rows
// beyond the sequence zero-filled) into a two-stage ring, rows padded by 16 bytes
// so that ldmatrix reads are conflict-free.  Per 16 positions a warp issues 32
// MMAs and 16 ldmatrix for 8 KB of cache: the kernel is left to wait for memory.
constexpr int ADT_STAGE_POS = 64;
constexpr int ADT_STAGES = 2;

template <typename TC>
struct Mma16;
template <>
struct Mma16<__half> {
  __device__ static uint32_t pack(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }
  __device__ static void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <>
struct Mma16<__nv_bfloat16> {
  __device__ static uint32_t pack(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  __device__ static void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16-byte copy, or 16 bytes of zeros when `valid` is false
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

template <typename TC, int HD>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_mma_kernel(const DecodeArgs a) {
  constexpr int ROW_B = HD * 2;
  constexpr int ROW_PAD = ROW_B + 16;
  constexpr int CHUNKS = ROW_B / 16;
  constexpr int TILE = ADT_STAGE_POS * ROW_PAD;       // one K or V tile of a stage
  constexpr int KSTEPS = HD / 16, DTILES = HD / 8;
  extern __shared__ __align__(16) uint8_t s_ring[];   // [stage][K tile | V tile]
  __shared__ long long s_row[ADT_STAGES][ADT_STAGE_POS];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int G = a.heads / a.kv_heads;
  const int seq_len = a.seq_lens[b];
  const TC* slab = static_cast<const TC*>(a.slab);
  const size_t row_elems = static_cast<size_t>(a.kv_heads) * HD;
  const size_t page_elems = static_cast<size_t>(a.blocks) * 2 * a.stride * row_elems;
  const size_t v_off = static_cast<size_t>(a.stride) * row_elems;

  // this split's positions, in whole stages
  const int stages_total = (seq_len + ADT_STAGE_POS - 1) / ADT_STAGE_POS;
  const int stages_per = (stages_total + a.splits - 1) / a.splits;
  const int p_begin = split * stages_per * ADT_STAGE_POS;
  const int p_end = min(seq_len, (split + 1) * stages_per * ADT_STAGE_POS);
  const int nstages = p_end > p_begin ? (p_end - p_begin + ADT_STAGE_POS - 1) / ADT_STAGE_POS : 0;

  // Q fragments: rows = heads (gid < G, else zero), scaled
  uint32_t qa0[KSTEPS], qa2[KSTEPS];
#pragma unroll
  for (int s = 0; s < KSTEPS; ++s) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (gid < G) {
      const size_t base = (static_cast<size_t>(b) * a.heads + kvh * G + gid) * HD + 16 * s + 2 * tig;
      v[0] = ld_elem(a.q, a.q_dtype, base) * a.scale;
      v[1] = ld_elem(a.q, a.q_dtype, base + 1) * a.scale;
      v[2] = ld_elem(a.q, a.q_dtype, base + 8) * a.scale;
      v[3] = ld_elem(a.q, a.q_dtype, base + 9) * a.scale;
    }
    qa0[s] = Mma16<TC>::pack(v[0], v[1]);
    qa2[s] = Mma16<TC>::pack(v[2], v[3]);
  }

  auto issue_stage = [&](int st_i) {
    const int slot = st_i % ADT_STAGES;
    const int p0 = p_begin + st_i * ADT_STAGE_POS;
    if (t < ADT_STAGE_POS) {
      const int pos = p0 + t;
      long long row = -1;
      if (pos < p_end) {
        const int pslot = pos / a.stride;
        const long long page = pslot < a.pages_per_seq ? a.page_ids[b * a.pages_per_seq + pslot] : -1;
        if (page < 0 || page >= a.page_count) {
          atomicOr(a.status, DEV_ERR_BOUNDS);
        } else {
          row = static_cast<long long>(static_cast<size_t>(page) * page_elems +
                                       ((static_cast<size_t>(a.block_index) * 2) * a.stride + pos % a.stride) * row_elems +
                                       static_cast<size_t>(kvh) * HD);
        }
      }
      s_row[slot][t] = row;
    }
    __syncthreads();
    uint8_t* kt = s_ring + slot * 2 * TILE;
    uint8_t* vt = kt + TILE;
    for (int i = t; i < ADT_STAGE_POS * CHUNKS; i += AD_THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const long long row = s_row[slot][r];
      const TC* src = slab + (row >= 0 ? row : 0) + c * 8;
      cp_async16_zfill(smem_u32(kt + r * ROW_PAD + c * 16), src, row >= 0);
      cp_async16_zfill(smem_u32(vt + r * ROW_PAD + c * 16), src + v_off, row >= 0);
    }
    cp_async_commit();
  };

  float m_run = -INFINITY, l_run = 0.f;  // head gid; l_run is this lane's share (its tig columns)
  float o[DTILES][2];                    // O[head gid][d = 8*j + 2*tig, +1]
#pragma unroll
  for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = 0.f;

  if (nstages > 0) issue_stage(0);
  for (int st_i = 0; st_i < nstages; ++st_i) {
    if (st_i + 1 < nstages) {
      issue_stage(st_i + 1);   // its barrier also says: stage st_i - 1's slot is no longer read
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();           // stage st_i has landed for everyone
    const int slot = st_i % ADT_STAGES;
    const uint32_t kt = smem_u32(s_ring + slot * 2 * TILE) + warp * 16 * ROW_PAD;
    const uint32_t vt = kt + TILE;
    const int p0 = p_begin + st_i * ADT_STAGE_POS + warp * 16;  // this warp's 16 positions

    // S[head][pos]: two n-tiles of 8 positions
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
    {
      const int mi = lane >> 3, r = lane & 7;  // matrix index and row this lane addresses
      const uint32_t base = kt + (8 * (mi >> 1) + r) * ROW_PAD + 16 * (mi & 1);
#pragma unroll
      for (int s = 0; s < KSTEPS; ++s) {
        uint32_t kb[4];
        ldmatrix_x4(base + 32 * s, kb);
        Mma16<TC>::mma(sc[0], qa0[s], 0u, qa2[s], 0u, kb[0], kb[1]);
        Mma16<TC>::mma(sc[1], qa0[s], 0u, qa2[s], 0u, kb[2], kb[3]);
      }
    }
    // online softmax for head gid over this lane's four positions, then across the tig lanes
    float pv[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float v = sc[j][e];
        if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
        if (p0 + 8 * j + 2 * tig + e >= p_end) v = -INFINITY;
        pv[j][e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float alpha = (m_new == -INFINITY) ? 1.f : __expf(m_run - m_new);
    float psum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p = (pv[j][e] == -INFINITY) ? 0.f : __expf(pv[j][e] - m_new);
        pv[j][e] = p;
        psum += p;
      }
    m_run = m_new;
    l_run = l_run * alpha + psum;
    const uint32_t pa0 = Mma16<TC>::pack(pv[0][0], pv[0][1]);
    const uint32_t pa2 = Mma16<TC>::pack(pv[1][0], pv[1][1]);
    // O[head][d] = O * alpha + P . V
    {
      const int mi = lane >> 3, r = lane & 7;
      const uint32_t base = vt + (8 * (mi & 1) + r) * ROW_PAD + 16 * (mi >> 1);
#pragma unroll
      for (int j = 0; j < DTILES; j += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(base + 16 * j, vb);
        float c0[4] = {o[j][0] * alpha, o[j][1] * alpha, 0.f, 0.f};
        float c1[4] = {o[j + 1][0] * alpha, o[j + 1][1] * alpha, 0.f, 0.f};
        Mma16<TC>::mma(c0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
        Mma16<TC>::mma(c1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
        o[j][0] = c0[0]; o[j][1] = c0[1];
        o[j + 1][0] = c1[0]; o[j + 1][1] = c1[1];
      }
    }
  }
  // this lane's share of the denominator -> the head's
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

  // merge the four warps (each saw different positions) through shared memory
  __syncthreads();  // the ring is free
  float* s_o = reinterpret_cast<float*>(s_ring);            // [warp][G][HD]
  float* s_ml = s_o + 4 * AD_MAXG * HD;                       // [warp][G][2]
  if (gid < G) {
#pragma unroll
    for (int j = 0; j < DTILES; ++j) {
      s_o[(warp * AD_MAXG + gid) * HD + 8 * j + 2 * tig] = o[j][0];
      s_o[(warp * AD_MAXG + gid) * HD + 8 * j + 2 * tig + 1] = o[j][1];
    }
    if (tig == 0) {
      s_ml[(warp * AD_MAXG + gid) * 2] = m_run;
      s_ml[(warp * AD_MAXG + gid) * 2 + 1] = l_run;
    }
  }
  __syncthreads();
  float* out = a.partial + ((static_cast<size_t>(b) * a.kv_heads + kvh) * a.splits + split) * G * (HD + 2);
  for (int i = t; i < G * HD; i += AD_THREADS) {
    const int g = i / HD, d = i % HD;
    float M = -INFINITY;
    for (int w = 0; w < 4; ++w) M = fmaxf(M, s_ml[(w * AD_MAXG + g) * 2]);
    float acc = 0.f, L = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float m = s_ml[(w * AD_MAXG + g) * 2];
      if (m != -INFINITY) {
        const float f = __expf(m - M);
        acc += s_o[(w * AD_MAXG + g) * HD + d] * f;
        L += s_ml[(w * AD_MAXG + g) * 2 + 1] * f;
      }
    }
    out[g * (HD + 2) + d] = acc;
    if (d == 0) {
      out[g * (HD + 2) + HD] = M;
      out[g * (HD + 2) + HD + 1] = L;
    }
  }
}

// Merges the splits: out[b, head, d] = sum_s acc_s * exp(m_s - M) / sum_s l_s * exp(m_s - M).
__global__ void __launch_bounds__(128)
attn_decode_merge_kernel(const float* __restrict__ partial, int splits, int G, int hd, int heads, int kv_heads,
                         void* __restrict__ out, int out_dtype) {
  const int head = blockIdx.x, b = blockIdx.y;
  const int kvh = head / G, g = head % G;
  const float* base = partial + ((static_cast<size_t>(b) * kv_heads + kvh) * splits) * G * (hd + 2) + g * (hd + 2);
  const size_t sstride = static_cast<size_t>(G) * (hd + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * sstride + hd]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = base[s * sstride + hd];
    if (m != -INFINITY) L += base[s * sstride + hd + 1] * __expf(m - M);
  }
  for (int d = threadIdx.x; d < hd; d += 128) {
    float o = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = base[s * sstride + hd];
      if (m != -INFINITY) o += base[s * sstride + d] * __expf(m - M);
    }
    st_elem(out, out_dtype, (static_cast<size_t>(b) * heads + head) * hd + d, L > 0.f ? o / L : 0.f);
  }
}

int decode_splits(int bs, int kv_heads, int max_seq_len) {
  // about six CTAs per SM (each holds 64-130 KB of shared-memory tiles at most
  // three deep, and the steps of one CTA are serial), but no split shorter than
  // one 128-position step
  const int base = bs * kv_heads;
  int splits = (6 * sm_count() + base - 1) / base;
  const int most = (max_seq_len + AD_THREADS - 1) / AD_THREADS;
  if (splits > most) splits = most;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  return splits;
}

template <typename TC, int HD>
int launch_decode_mma(const DecodeArgs& a, dim3 grid, cudaStream_t st) {
  constexpr int RING = ADT_STAGES * 2 * ADT_STAGE_POS * (HD * 2 + 16);
  constexpr int MERGE = (4 * AD_MAXG * HD + 4 * AD_MAXG * 2) * 4;
  constexpr int SMEM = RING > MERGE ? RING : MERGE;
  auto kern = attn_decode_mma_kernel<TC, HD>;
  static bool configured[16] = {};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev] = true;
  }
  kern<<<grid, AD_THREADS, SMEM, st>>>(a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

template <typename TC, int HD>
int launch_decode(const DecodeArgs& a, dim3 grid, cudaStream_t st) {
  constexpr int SMEM = 2 * AD_THREADS * (HD * static_cast<int>(sizeof(TC)) + 16);
  auto kern = attn_decode_kernel<TC, HD>;
  static bool configured[16] = {};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev] = true;
  }
  kern<<<grid, AD_THREADS, SMEM, st>>>(a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

bool dtype_ok(int dt) { return dt == B200MOE_DT_F32 || dt == B200MOE_DT_F16 || dt == B200MOE_DT_BF16; }

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_rms_norm(const void* x, int x_dtype, const float* weight, int64_t rows, int32_t d, float eps,
                     void* y, int y_dtype, void* stream) {
  B200_REQUIRE(rows >= 0 && d > 0, "rms_norm: bad sizes");
  if (rows == 0) return B200MOE_OK;
  B200_REQUIRE(x && weight && y && dtype_ok(x_dtype) && dtype_ok(y_dtype), "rms_norm: bad argument");
  rms_norm_rows_kernel<<<static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      x, x_dtype, weight, d, eps, y, y_dtype);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

int b200moe_attn_rope_kv_write(void* q, const void* k, const void* v, void* k_out, void* v_out, int io_dtype,
                               void* slab, int cache_dtype, const b200moe_kv_cache_t* cache,
                               int32_t block_index, const int32_t* positions, const int32_t* page_ids,
                               const float* freqs, int32_t tokens, int32_t tokens_per_seq,
                               int32_t pages_per_seq, int32_t heads, void* stream) {
  B200_REQUIRE(cache != nullptr, "attn_rope_kv_write: NULL cache geometry");
  B200_REQUIRE(tokens >= 0 && tokens_per_seq >= 1 && pages_per_seq >= 1 && heads >= 1, "attn_rope_kv_write: bad sizes");
  if (tokens == 0) return B200MOE_OK;
  B200_REQUIRE(q && k && v && slab && positions && page_ids && freqs, "attn_rope_kv_write: NULL buffer");
  B200_REQUIRE((k_out == nullptr) == (v_out == nullptr), "attn_rope_kv_write: k_out and v_out go together");
  B200_REQUIRE(dtype_ok(io_dtype) && dtype_ok(cache_dtype), "attn_rope_kv_write: unknown dtype");
  B200_REQUIRE(cache->head_dim % 2 == 0 && cache->kv_heads >= 1 && cache->stride >= 1 && cache->blocks >= 1 &&
                   block_index >= 0 && block_index < cache->blocks && cache->page_count >= 1,
               "attn_rope_kv_write: bad cache geometry");
  B200_REQUIRE(tokens % tokens_per_seq == 0, "attn_rope_kv_write: tokens must be whole sequences");
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  RopeArgs a;
  a.q = q; a.k = k; a.v = v; a.k_out = k_out; a.v_out = v_out; a.io_dtype = io_dtype;
  a.slab = slab; a.cache_dtype = cache_dtype; a.positions = positions; a.page_ids = page_ids; a.freqs = freqs;
  a.tokens = tokens; a.tokens_per_seq = tokens_per_seq; a.pages_per_seq = pages_per_seq;
  a.page_count = cache->page_count; a.heads = heads; a.kv_heads = cache->kv_heads; a.hd = cache->head_dim;
  a.stride = cache->stride; a.blocks = cache->blocks; a.block_index = block_index; a.status = status;
  rope_kv_write_kernel<<<tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

size_t b200moe_attn_decode_scratch_bytes(const b200moe_kv_cache_t* cache, int32_t bs, int32_t heads,
                                         int32_t max_seq_len) {
  if (cache == nullptr || bs <= 0 || heads <= 0 || cache->kv_heads <= 0 || heads % cache->kv_heads != 0) return 0;
  const int splits = decode_splits(bs, cache->kv_heads, max_seq_len);
  return static_cast<size_t>(bs) * heads * splits * (cache->head_dim + 2) * sizeof(float);
}

int b200moe_attn_decode(const void* q, int q_dtype, const void* slab, int cache_dtype,
                        const b200moe_kv_cache_t* cache, int32_t block_index, const int32_t* page_ids,
                        const int32_t* seq_lens, int32_t bs, int32_t pages_per_seq, int32_t heads,
                        int32_t max_seq_len, float scale, float softcap, void* out, int out_dtype,
                        void* scratch, size_t scratch_bytes, void* stream) {
  B200_REQUIRE(cache != nullptr, "attn_decode: NULL cache geometry");
  B200_REQUIRE(bs >= 0 && pages_per_seq >= 1 && heads >= 1 && max_seq_len >= 1, "attn_decode: bad sizes");
  if (bs == 0) return B200MOE_OK;
  B200_REQUIRE(q && slab && page_ids && seq_lens && out && scratch, "attn_decode: NULL buffer");
  B200_REQUIRE(dtype_ok(q_dtype) && dtype_ok(cache_dtype) && dtype_ok(out_dtype), "attn_decode: unknown dtype");
  B200_REQUIRE(cache->kv_heads >= 1 && heads % cache->kv_heads == 0 && heads / cache->kv_heads <= AD_MAXG,
               "attn_decode: heads (%d) must be 1..8 times the kv heads (%d)", heads, cache->kv_heads);
  B200_REQUIRE(cache->head_dim == 64 || cache->head_dim == 128, "attn_decode: head_dim %d (64 and 128 are built)",
               cache->head_dim);
  B200_REQUIRE(block_index >= 0 && block_index < cache->blocks && cache->stride >= 1, "attn_decode: bad block index");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(slab) & 15) == 0, "attn_decode: page slab must be 16-byte aligned");
  const size_t need = b200moe_attn_decode_scratch_bytes(cache, bs, heads, max_seq_len);
  if (scratch_bytes < need) {
    set_error("attn_decode: scratch needs %zu bytes, got %zu", need, scratch_bytes);
    return B200MOE_ERR_WORKSPACE;
  }
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DecodeArgs a;
  a.q = q; a.q_dtype = q_dtype; a.slab = slab; a.page_ids = page_ids; a.seq_lens = seq_lens;
  a.partial = static_cast<float*>(scratch);
  a.bs = bs; a.heads = heads; a.kv_heads = cache->kv_heads; a.hd = cache->head_dim; a.stride = cache->stride;
  a.blocks = cache->blocks; a.block_index = block_index; a.pages_per_seq = pages_per_seq;
  a.page_count = cache->page_count; a.splits = decode_splits(bs, cache->kv_heads, max_seq_len);
  a.scale = scale; a.softcap = softcap; a.status = status;
  const dim3 grid(a.splits, a.kv_heads, bs);
  const int hd = cache->head_dim;
  int rc;
  if (cache_dtype == B200MOE_DT_F32)
    rc = hd == 64 ? launch_decode<float, 64>(a, grid, st) : launch_decode<float, 128>(a, grid, st);
  else if (cache_dtype == B200MOE_DT_F16)
    rc = hd == 64 ? launch_decode_mma<__half, 64>(a, grid, st) : launch_decode_mma<__half, 128>(a, grid, st);
  else
    rc = hd == 64 ? launch_decode_mma<__nv_bfloat16, 64>(a, grid, st)
                  : launch_decode_mma<__nv_bfloat16, 128>(a, grid, st);
  if (rc) return rc;
  attn_decode_merge_kernel<<<dim3(heads, bs), 128, 0, st>>>(a.partial, a.splits, heads / cache->kv_heads, hd, heads,
                                                            cache->kv_heads, out, out_dtype);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

}  // extern "C"
