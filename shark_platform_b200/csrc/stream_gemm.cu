// Weight-streaming grouped expert GEMM for the decode regime (few tokens per
// expert, HBM-bound).
//
// Orientation is "swap-AB": a 16x16 tile of *weights* is the A operand of
// mma.sync.m16n8k16 and 8 tokens form the N dimension, so an expert with 1..8
// tokens costs one MMA column block and the quantised weights are read from HBM
// exactly once.  A producer warp streams the quantised weight tiles, their
// block scales and the tokens' activation rows into a shared-memory ring with
// TMA (128-byte swizzle); eight consumer warps dequantise straight from the
// staged bytes into MMA fragments in registers (no shared-memory round trip
// for the dequantised values) and accumulate in fp32.
//
// One CTA per SM, persistent over work items (expert, row tile, k split, token
// chunk).  Per stage a CTA holds two "row sets" of 64 weight rows x 256 k:
// gate rows and up rows of the same output columns (fused SiLU/GELU-gated
// product in the epilogue), or 128 consecutive rows of the down matrix.
// Consumer warp (w, kh): rows 16w..16w+15 of both sets, k half kh of the
// stage; the two k halves are added through shared memory at the end of an item.
#include "common.cuh"

namespace b200moe {

namespace {

constexpr int KT = 256;   // reduction elements per stage
constexpr int MAX_E = 64;

struct StreamArgs {
  const int32_t* seg;
  int E, N, K;
  int ntiles;           // row tiles per expert
  int ksplit;           // k partitions per row tile
  int stages_per_item;  // (K / KT) / ksplit
  int P;                // rows of the activation / output arrays
  int act;
  int out_kperm;        // gate/up only: permute output columns for a Q4_K down matrix
  void* out;
  int32_t* status;
  // Q8_0 only: scales transposed to [K/256][rows][8] (16 bytes per row and
  // stage, consecutive rows contiguous); NULL = fetch them as 16-byte TMA rows
  const uint8_t* st0;
  const uint8_t* st1;
  long long total_rows;  // E * N
};

// Untiled bulk copy global -> shared (both 16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// RW = row warps per k part: 4 (64 rows per set) or 7 (112 rows per set: 112-row
// tiles divide ffn sizes with a factor 7 (14336 = 128 x 112) into a number of
// work items that fills the last wave of SMs).  KH = k parts of a stage handled
// by different warps (the parts are added through shared memory at the end of an
// item).  Consumer warps = RW * KH: (4,2) = 8 and (7,1) = 7 are the narrow
// geometries, (4,4) = 16 and (7,2) = 14 the wide ones — the same tiles with twice
// the warps, for layouts whose dequantisation is instruction-bound.
template <int LAYOUT, int S, int RW, int KH_>
struct Cfg {
  static constexpr int SET_ROWS = 16 * RW;
  static constexpr int KH = KH_;               // k parts handled by different warps
  static constexpr int ACTIVE = RW * KH;       // consumer warps
  static constexpr int GROUP = RW * 32;        // threads of one k part
  static constexpr int THREADS = (ACTIVE + 1) * 32;  // + the TMA producer warp
  static constexpr int MT = 8 * S;  // tokens per chunk
  // bytes of one row set of quantised values per stage
  static constexpr int WSET = LAYOUT == B200MOE_LAYOUT_Q8_0   ? SET_ROWS * KT
                              : LAYOUT == B200MOE_LAYOUT_Q4_K ? SET_ROWS * KT / 2
                                                              : SET_ROWS * KT * 2;
  // scale bytes per row per stage
  static constexpr int SROW = LAYOUT == B200MOE_LAYOUT_Q8_0 ? 16 : LAYOUT == B200MOE_LAYOUT_Q4_K ? 32 : 0;
  static constexpr int SSET = SET_ROWS * SROW;
  static constexpr int XBOX = MT * 128;
  static constexpr int OFF_X = 2 * WSET;
  static constexpr int OFF_S = OFF_X + 4 * XBOX;
  static constexpr int STAGE = (OFF_S + 2 * SSET + 1023) / 1024 * 1024;
  // floats per thread per reduce round (fewer with more source parts: each part has a buffer)
  static constexpr int RED_FLOATS = KH > 2 ? 8 : (8 * S < 32 ? 8 * S : 32);
  static constexpr int RED_BYTES = (KH > 1 ? KH - 1 : 1) * GROUP * RED_FLOATS * 4;  // one buffer per source part
  static constexpr int BUDGET = 232448 - 1024 - RED_BYTES - 256;
  static constexpr int STAGES_RAW = BUDGET / STAGE;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SMEM = 1024 + STAGES * STAGE + RED_BYTES + 256;
  static_assert(STAGE % 1024 == 0, "stage must keep 1024-byte alignment for the swizzle");
  static_assert(STAGES >= 2, "pipeline too shallow");
};

__device__ __forceinline__ int rho(int g) { return (g >> 1) | ((g & 1) << 2); }

// half2 with both halves = half `sel` (0 = low, 1 = high) of `v`
__device__ __forceinline__ __half2 bcast_half(uint32_t v, int sel) {
  return u32_as_h2(__byte_perm(v, v, sel ? 0x3232 : 0x1010));
}

template <int LAYOUT, int NMAT, int S, int RW, int KH_>
__global__ void __launch_bounds__((RW * KH_ + 1) * 32, 1)
stream_gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                   const __grid_constant__ CUtensorMap tm_s0, const __grid_constant__ CUtensorMap tm_s1,
                   const __grid_constant__ CUtensorMap tm_x8, const __grid_constant__ CUtensorMap tm_x16,
                   const __grid_constant__ CUtensorMap tm_x32, const __grid_constant__ CUtensorMap tm_x64,
                   const StreamArgs args) {
  using C = Cfg<LAYOUT, S, RW, KH_>;
  constexpr int STAGES = C::STAGES;
  constexpr int SET_ROWS = C::SET_ROWS;
  constexpr int KH = C::KH;
  constexpr int GROUP = C::GROUP;
  constexpr int SPANS = 4 / KH;  // 64-k spans of a stage per warp
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_seg[MAX_E + 1];
  __shared__ int s_prefix[MAX_E + 1];
  __shared__ int s_abort;
  __shared__ int s_exit;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t red_base = smem_base + STAGES * C::STAGE;
  const uint32_t bar_base = red_base + C::RED_BYTES;  // full[STAGES], empty[STAGES]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    s_exit = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), C::ACTIVE);
    }
    fence_mbar_init();
    int run = 0;
    for (int e = 0; e < args.E; ++e) {
      const int a = args.seg[e], b = args.seg[e + 1];
      s_seg[e] = a;
      s_prefix[e] = run;
      const int chunks = (b - a + C::MT - 1) / C::MT;
      run += chunks * args.ntiles * args.ksplit;
    }
    s_seg[args.E] = args.seg[args.E];
    s_prefix[args.E] = run;
  }
  __syncthreads();
  const int total_items = s_prefix[args.E];
  volatile int* abort_flag = &s_abort;

  auto decode = [&](int item, int& e, int& tile, int& kc, int& row0, int& rows) {
    e = 0;
    while (item >= s_prefix[e + 1]) ++e;
    const int local = item - s_prefix[e];
    const int m = s_seg[e + 1] - s_seg[e];
    const int chunks = (m + C::MT - 1) / C::MT;
    const int tc = local % chunks;
    const int rest = local / chunks;
    kc = rest % args.ksplit;
    tile = rest / args.ksplit;
    row0 = s_seg[e] + tc * C::MT;
    rows = min(C::MT, s_seg[e + 1] - row0);
  };

  if (warp == C::ACTIVE) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t n = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int e, tile, kc, row0, rows;
        decode(item, e, tile, kc, row0, rows);
        const int n0 = tile * (NMAT == 2 ? SET_ROWS : 2 * SET_ROWS);
        // token boxes no taller than the segment needs (each box row is one TMA request)
        const CUtensorMap* tx = rows <= 8 ? &tm_x8 : rows <= 16 ? &tm_x16 : rows <= 32 ? &tm_x32 : &tm_x64;
        const int xrows = rows <= 8 ? 8 : rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
        const uint32_t tx_bytes = 2 * C::WSET + 2 * C::SSET + 4 * xrows * 128;
        for (int st = 0; st < args.stages_per_item; ++st, ++n) {
          const int slot = n % STAGES;
          const uint32_t phase = (n / STAGES) & 1u;
          if (!mbar_wait(empty_bar(slot), phase ^ 1u, abort_flag, args.status)) { ok = false; break; }
          fence_proxy_async_smem();
          const uint32_t sb = smem_base + slot * C::STAGE;
          const uint32_t fb = full_bar(slot);
          mbar_expect_tx(fb, tx_bytes);
          const int k0 = (kc * args.stages_per_item + st) * KT;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const CUtensorMap* tw = (NMAT == 2 && r == 1) ? &tm_w1 : &tm_w0;
            const CUtensorMap* ts = (NMAT == 2 && r == 1) ? &tm_s1 : &tm_s0;
            const int grow = e * args.N + n0 + (NMAT == 2 ? 0 : SET_ROWS * r);
            if constexpr (LAYOUT == B200MOE_LAYOUT_Q8_0) {
              tma_load_2d(sb + r * C::WSET, tw, k0, grow, fb);
              tma_load_2d(sb + r * C::WSET + SET_ROWS * 128, tw, k0 + 128, grow, fb);
              if (args.st0 != nullptr) {
                const uint8_t* sp = (NMAT == 2 && r == 1) ? args.st1 : args.st0;
                bulk_load(sb + C::OFF_S + r * C::SSET,
                          sp + (static_cast<long long>(k0 / KT) * args.total_rows + grow) * 16,
                          C::SSET, fb);
              } else {
                tma_load_2d(sb + C::OFF_S + r * C::SSET, ts, (k0 / 32) * 2, grow, fb);
              }
            } else if constexpr (LAYOUT == B200MOE_LAYOUT_Q4_K) {
              tma_load_2d(sb + r * C::WSET, tw, k0 / 2, grow, fb);
              tma_load_2d(sb + C::OFF_S + r * C::SSET, ts, (k0 / 32) * 4, grow, fb);
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                tma_load_2d(sb + r * C::WSET + c * (SET_ROWS * 128), tw, (k0 + 64 * c) * 2, grow, fb);
            }
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tma_load_2d(sb + C::OFF_X + c * C::XBOX, tx, (k0 + 64 * c) * 2, row0, fb);
        }
      }
      // Do not leave while copies may still land in this CTA's shared memory.
      const uint32_t issued = n;
      const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
      for (uint32_t i = first; i < issued; ++i)
        mbar_wait(full_bar(i % STAGES), (i / STAGES) & 1u, abort_flag, args.status);
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int w = warp % RW, kh = warp / RW;
  const int g = lane >> 2, t = lane & 3;
  const int rg = rho(g);
  const int ctid = tid % GROUP;  // index within a k-part group
  uint32_t n = 0;

  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    int e, tile, kc, row0, rows;
    decode(item, e, tile, kc, row0, rows);
    const int s_act = (rows + 7) >> 3;
    float acc[2][S][4];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int s = 0; s < S; ++s)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][s][c] = 0.f;

    for (int st = 0; st < args.stages_per_item; ++st, ++n) {
      const int slot = n % STAGES;
      const uint32_t phase = (n / STAGES) & 1u;
      if (!mbar_wait_warp(full_bar(slot), phase, abort_flag, args.status)) break;
      const uint32_t sb = smem_base + slot * C::STAGE;

      if constexpr (LAYOUT == B200MOE_LAYOUT_Q8_0) {
        uint32_t sc[2][2][SPANS];  // [set][row half][the two block scales of each of the warp's spans]
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint32_t srow = sb + C::OFF_S + r * C::SSET + (16 * w + rg) * 16 + kh * SPANS * 4;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if constexpr (SPANS == 4) lds128(srow + hf * 8 * 16, sc[r][hf]);
            else if constexpr (SPANS == 2) lds64(srow + hf * 8 * 16, sc[r][hf]);
            else sc[r][hf][0] = lds32(srow + hf * 8 * 16);
          }
        }
#pragma unroll
        for (int spi = 0; spi < SPANS; ++spi) {
          const int sp = SPANS * kh + spi;  // 64-k span of the stage
          const int cb = (sp & 1) * 4;
          uint32_t alo[2][2][4], ahi[2][2][4];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint32_t wbase = sb + r * C::WSET + (sp >> 1) * (SET_ROWS * 128) +
                                   (16 * w + rg) * 128 + (((cb + t) ^ rg) << 4);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              uint32_t q[4];
              lds128(wbase + hf * 8 * 128, q);
              const uint32_t sw = sc[r][hf][spi];
              const __half2 scale = bcast_half(sw, t >> 1);
#pragma unroll
              for (int j = 0; j < 4; ++j) dequant_q8x4(q[j], scale, alo[r][hf][j], ahi[r][hf][j]);
            }
          }
#pragma unroll
          for (int s = 0; s < S; ++s) {
            if (s < s_act) {
              const uint32_t xrow = sb + C::OFF_X + sp * C::XBOX + (8 * s + g) * 128;
              uint32_t b[8];
              lds128(xrow + (((2 * t) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[0]));
              lds128(xrow + (((2 * t + 1) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[4]));
#pragma unroll
              for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < 2; ++r)
                  mma_16816(acc[r][s], alo[r][0][j], alo[r][1][j], ahi[r][0][j], ahi[r][1][j],
                            b[2 * j], b[2 * j + 1]);
            }
          }
        }
      } else if constexpr (LAYOUT == B200MOE_LAYOUT_F16) {
        // dense fp16 weights: one 128-byte box per 64-k span, fragments are the
        // staged values themselves
#pragma unroll
        for (int spi = 0; spi < SPANS; ++spi) {
          const int sp = SPANS * kh + spi;
          uint32_t a[2][2][8];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const uint32_t wrow = sb + r * C::WSET + sp * (SET_ROWS * 128) +
                                    (16 * w + rg + 8 * hf) * 128;
              lds128(wrow + (((2 * t) ^ rg) << 4), *reinterpret_cast<uint32_t(*)[4]>(&a[r][hf][0]));
              lds128(wrow + (((2 * t + 1) ^ rg) << 4), *reinterpret_cast<uint32_t(*)[4]>(&a[r][hf][4]));
            }
          }
#pragma unroll
          for (int s = 0; s < S; ++s) {
            if (s < s_act) {
              const uint32_t xrow = sb + C::OFF_X + sp * C::XBOX + (8 * s + g) * 128;
              uint32_t b[8];
              lds128(xrow + (((2 * t) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[0]));
              lds128(xrow + (((2 * t + 1) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[4]));
#pragma unroll
              for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < 2; ++r)
                  mma_16816(acc[r][s], a[r][0][2 * j], a[r][1][2 * j], a[r][0][2 * j + 1],
                            a[r][1][2 * j + 1], b[2 * j], b[2 * j + 1]);
            }
          }
        }
      } else {
        // Q4_K: one 128-byte box row = 256 k = one super-block; a 64-k span is
        // 32 bytes; thread t owns 8 bytes = 16 quants of sub-block 2*sp + (t>>1).
#pragma unroll
        for (int spi = 0; spi < SPANS; ++spi) {
          const int sp = SPANS * kh + spi;
          uint32_t a[2][2][4][2];  // [set][row half][mma j][lo,hi]
#pragma unroll
          for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int row = 16 * w + rg + 8 * hf;
              // bytes sp*32 + t*8 .. +8 of the row: chunk 2*sp + (t>>1), half (t&1)
              const uint32_t addr = sb + r * C::WSET + row * 128 +
                                    (((2 * sp + (t >> 1)) ^ rg) << 4) + 8 * (t & 1);
              uint32_t q[2];
              lds64(addr, q);
              const uint32_t sm =
                  lds32(sb + C::OFF_S + r * C::SSET + row * 32 + (2 * sp + (t >> 1)) * 4);
              const __half2 ds = bcast_half(sm, 0), dm = bcast_half(sm, 1);
              uint32_t o0[4], o1[4];
              dequant_q4x8(q[0], ds, dm, o0);
              dequant_q4x8(q[1], ds, dm, o1);
              // word q[0] covers k 0..7 of the thread's 16, q[1] covers 8..15;
              // mma j uses the thread's k 4j..4j+3 in permuted order, i.e. the
              // pairs (2 per half-word) numbered 2j and 2j+1 of the 8 produced.
              a[r][hf][0][0] = o0[0]; a[r][hf][0][1] = o0[1];
              a[r][hf][1][0] = o0[2]; a[r][hf][1][1] = o0[3];
              a[r][hf][2][0] = o1[0]; a[r][hf][2][1] = o1[1];
              a[r][hf][3][0] = o1[2]; a[r][hf][3][1] = o1[3];
            }
          }
#pragma unroll
          for (int s = 0; s < S; ++s) {
            if (s < s_act) {
              const uint32_t xrow = sb + C::OFF_X + sp * C::XBOX + (8 * s + g) * 128;
              uint32_t b[8];
              lds128(xrow + (((2 * t) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[0]));
              lds128(xrow + (((2 * t + 1) ^ g) << 4), *reinterpret_cast<uint32_t(*)[4]>(&b[4]));
#pragma unroll
              for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < 2; ++r)
                  mma_16816(acc[r][s], a[r][0][j][0], a[r][1][j][0], a[r][0][j][1], a[r][1][j][1],
                            b[2 * j], b[2 * j + 1]);
            }
          }
        }
      }
      fence_proxy_async_smem();  // reads done before TMA may refill the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(slot));
    }

    if constexpr (KH > 1) {
      // ---- add the k parts: parts 1.. hand their sums to part 0, each through
      // its own buffer
      constexpr int TOTAL = 8 * S;
      constexpr int ROUNDS = TOTAL / C::RED_FLOATS;
      constexpr int BUF = GROUP * C::RED_FLOATS;  // floats of one part's buffer
      float* accf = &acc[0][0][0];
      float* red = reinterpret_cast<float*>(smem_raw + (red_base - smem_u32(smem_raw)));
#pragma unroll
      for (int rd = 0; rd < ROUNDS; ++rd) {
        if (kh > 0) {
#pragma unroll
          for (int i = 0; i < C::RED_FLOATS; ++i)
            red[(kh - 1) * BUF + i * GROUP + ctid] = accf[rd * C::RED_FLOATS + i];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(KH * GROUP) : "memory");
        if (kh == 0) {
#pragma unroll
          for (int src = 0; src < KH - 1; ++src)
#pragma unroll
            for (int i = 0; i < C::RED_FLOATS; ++i)
              accf[rd * C::RED_FLOATS + i] += red[src * BUF + i * GROUP + ctid];
          // one thread decides for all consumers whether the CTA gives up, so
          // that every warp leaves the item loop at the same barrier
          if (rd == ROUNDS - 1 && ctid == 0) s_exit = *abort_flag;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(KH * GROUP) : "memory");
      }
      if (s_exit) break;
      if (kh != 0) continue;
    } else {
      if (*abort_flag) break;  // no barriers between consumer warps in this geometry
    }

    // ---- epilogue
    const int seg_end = row0 + rows;
#pragma unroll
    for (int s = 0; s < S; ++s) {
      if (s >= s_act) continue;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = row0 + 8 * s + 2 * t + (c & 1);
        if (tok >= seg_end) continue;
        const int rsub = 16 * w + rg + 8 * (c >> 1);
        if constexpr (NMAT == 2) {
          const float gt = acc[0][s][c], up = acc[1][s][c];
          const float a = args.act == B200MOE_ACT_SILU ? silu_f(gt) : gelu_erf_f(gt);
          int col = tile * SET_ROWS + rsub;
          if (args.out_kperm) col = (col & ~7) | ((col & 3) << 1) | ((col >> 2) & 1);
          static_cast<__half*>(args.out)[static_cast<size_t>(tok) * args.N + col] =
              to_half_sat(a * up, args.status);
        } else {
          float* outp = static_cast<float*>(args.out) +
                        static_cast<size_t>(kc) * args.P * args.N +
                        static_cast<size_t>(tok) * args.N + tile * (2 * SET_ROWS) + rsub;
          outp[0] = acc[0][s][c];
          outp[SET_ROWS] = acc[1][s][c];
        }
      }
    }
  }
}

template <int LAYOUT, int NMAT, int S, int RW, int KH>
int launch_t(const CUtensorMap* maps, const StreamArgs& a, cudaStream_t st) {
  using C = Cfg<LAYOUT, S, RW, KH>;
  auto kern = stream_gemm_kernel<LAYOUT, NMAT, S, RW, KH>;
  static bool configured[16] = {};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    configured[dev] = true;
  }
  kern<<<sm_count(), C::THREADS, C::SMEM, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                                             maps[6], maps[7], a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

template <int LAYOUT, int NMAT, int RW, int KH>
int launch_s(int S, const CUtensorMap* maps, const StreamArgs& a, cudaStream_t st) {
  switch (S) {
    case 1: return launch_t<LAYOUT, NMAT, 1, RW, KH>(maps, a, st);
    case 2: return launch_t<LAYOUT, NMAT, 2, RW, KH>(maps, a, st);
    case 4: return launch_t<LAYOUT, NMAT, 4, RW, KH>(maps, a, st);
    default: return launch_t<LAYOUT, NMAT, 8, RW, KH>(maps, a, st);
  }
}

// 64-row sets with four k parts (16 consumer warps), chunks of up to 32 tokens
template <int LAYOUT, int NMAT>
int launch_w(int S, const CUtensorMap* maps, const StreamArgs& a, cudaStream_t st) {
  switch (S) {
    case 1: return launch_t<LAYOUT, NMAT, 1, 4, 4>(maps, a, st);
    case 2: return launch_t<LAYOUT, NMAT, 2, 4, 4>(maps, a, st);
    default: return launch_t<LAYOUT, NMAT, 4, 4, 4>(maps, a, st);
  }
}

// Twice the consumer warps on the same tiles (b200moe_set_stream_wide): -1 = for
// every quantised layout (measured at 32 tokens: Q4_K 0.354 -> 0.322 ms, Q8_0
// 0.317 -> 0.306 ms per layer; the kernel is bound by instruction issue, not by
// bytes, below that), 0 = never, 1 = always.  Chunks of more than 32 tokens keep
// the narrow geometry (registers); dense fp16 weights have no wide instance.
int g_stream_wide = -1;

bool use_wide(int layout, int S) {
  if (S > 4) return false;
  if (g_stream_wide >= 0) return g_stream_wide != 0;
  return layout == B200MOE_LAYOUT_Q4_K || layout == B200MOE_LAYOUT_Q8_0;
}

int weight_maps(const b200moe_weight_t* w, CUtensorMap* tw, CUtensorMap* ts, int SET_ROWS = 64) {
  const uint64_t rows = static_cast<uint64_t>(w->experts) * w->rows;
  if (w->layout == B200MOE_LAYOUT_Q8_0) {
    if (int rc = make_tmap_2d(tw, w->qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, w->cols, SET_ROWS,
                              128, true))
      return rc;
    return make_tmap_2d(ts, w->d, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, w->cols / 32 * 2,
                        SET_ROWS, 16, false);
  }
  if (w->layout == B200MOE_LAYOUT_F16) {
    *ts = CUtensorMap{};
    return make_tmap_2d(tw, w->qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows,
                        static_cast<uint64_t>(w->cols) * 2, SET_ROWS, 128, true);
  }
  if (int rc = make_tmap_2d(tw, w->qs, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, w->cols / 2,
                            SET_ROWS, 128, true))
    return rc;
  return make_tmap_2d(ts, w->sub, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, w->cols / 32 * 4,
                      SET_ROWS, 32, false);
}

// Token-row tensor maps with box heights 8, 16, 32 and 64 (maps[4..7]); heights
// above the kernel's chunk size 8*S are never selected and alias the largest valid one.
int token_maps(CUtensorMap* maps, const void* x, int pairs, uint64_t row_bytes, int S) {
  const int heights[4] = {8, 16, 32, 64};
  for (int i = 0; i < 4; ++i) {
    const int hgt = heights[i] <= 8 * S ? heights[i] : 8 * S;
    if (int rc = make_tmap_2d_sw(&maps[4 + i], x, pairs, row_bytes, hgt, 128, 128)) return rc;
  }
  return B200MOE_OK;
}

int pick_s(int max_segment) {
  if (max_segment <= 8) return 1;
  if (max_segment <= 16) return 2;
  if (max_segment <= 32) return 4;
  return 8;
}

int check_weight(const b200moe_weight_t* w, const char* name) {
  B200_REQUIRE(w->layout == B200MOE_LAYOUT_Q8_0 || w->layout == B200MOE_LAYOUT_Q4_K ||
                   w->layout == B200MOE_LAYOUT_F16,
               "stream kernel: %s layout %d unsupported", name, w->layout);
  B200_REQUIRE(w->cols % KT == 0, "stream kernel: %s cols (%d) must be a multiple of 256", name,
               w->cols);
  B200_REQUIRE(w->experts >= 1 && w->experts <= MAX_E, "stream kernel: %s experts out of range",
               name);
  B200_REQUIRE(w->qs != nullptr, "stream kernel: %s has no data", name);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(w->qs) & 15) == 0, "stream kernel: %s qs misaligned",
               name);
  if (w->layout == B200MOE_LAYOUT_Q8_0)
    B200_REQUIRE(w->d != nullptr && (reinterpret_cast<uintptr_t>(w->d) & 15) == 0,
                 "stream kernel: %s scales missing or misaligned", name);
  else if (w->layout == B200MOE_LAYOUT_Q4_K)
    B200_REQUIRE(w->sub != nullptr && (reinterpret_cast<uintptr_t>(w->sub) & 15) == 0,
                 "stream kernel: %s sub-block scales missing or misaligned", name);
  return B200MOE_OK;
}

}  // namespace

int stream_down_ksplit(const b200moe_weight_t* down, int pairs) {
  const int stages = down->cols / KT;
  if (pairs > 1024) return 1;
  if (stages % 4 == 0 && stages >= 8) return 4;
  if (stages % 2 == 0 && stages >= 4) return 2;
  return 1;
}

int launch_stream_gate_up(const void* xs, const int32_t* seg, int pairs, int max_segment,
                          const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                          int out_kperm, void* a_out, cudaStream_t st) {
  if (int rc = check_weight(gate, "gate")) return rc;
  if (int rc = check_weight(up, "up")) return rc;
  B200_REQUIRE(gate->layout == up->layout && gate->rows == up->rows && gate->cols == up->cols &&
                   gate->experts == up->experts,
               "stream kernel: gate and up must have the same layout and shape");
  B200_REQUIRE(gate->rows % 64 == 0, "stream kernel: ffn (%d) must be a multiple of 64", gate->rows);
  if (pairs == 0) return B200MOE_OK;
  int S = pick_s(max_segment);
  // max_segment is an upper bound (the token count); with several experts a
  // segment of more than half of it is rare and then takes two passes: chunks
  // one size down mean a smaller stage (and sixteen consumer warps up to 64 tokens).
  if (gate->experts >= 4) {
    if (S == 4) S = 2;
    else if (S == 8 && max_segment <= 64) S = 4;
  }
  // Tile height: 64 rows per set, or 112 where that fills the last wave of SMs
  // better (e.g. ffn 14336: 1792 items = 12.1 waves vs 1024 items = 6.9 waves).
  // The 112-row geometry has room for 16-token chunks only; longer segments are
  // processed in several chunks, so it is used for short segments only.
  int set_rows = 64;
  if (gate->layout == B200MOE_LAYOUT_Q8_0 && gate->rows % 112 == 0 && max_segment <= 32) {
    const double sms = sm_count();
    const int active = pairs < gate->experts ? pairs : gate->experts;
    auto eff = [&](int rows) {
      const double items = static_cast<double>(active) * (gate->rows / rows);
      const double waves = (items + sms - 1) / sms;
      return items / (static_cast<long long>(waves) * sms);
    };
    if (eff(112) > eff(64) + 0.02) {
      set_rows = 112;
      if (S > 2) S = 2;
    }
  }
  CUtensorMap maps[8];
  if (int rc = weight_maps(gate, &maps[0], &maps[2], set_rows)) return rc;
  if (int rc = weight_maps(up, &maps[1], &maps[3], set_rows)) return rc;
  if (int rc = token_maps(maps, xs, pairs, static_cast<uint64_t>(gate->cols) * 2, S)) return rc;
  StreamArgs a{};
  a.seg = seg; a.E = gate->experts; a.N = gate->rows; a.K = gate->cols;
  a.ntiles = gate->rows / set_rows; a.ksplit = 1; a.stages_per_item = gate->cols / KT;
  a.P = pairs; a.act = act; a.out_kperm = out_kperm; a.out = a_out; a.status = device_status_ptr();
  if (gate->layout == B200MOE_LAYOUT_Q8_0 && gate->sub != nullptr && up->sub != nullptr) {
    a.st0 = static_cast<const uint8_t*>(gate->sub);
    a.st1 = static_cast<const uint8_t*>(up->sub);
  }
  a.total_rows = static_cast<long long>(gate->experts) * gate->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  const bool wide = use_wide(gate->layout, S);
  if (set_rows == 112) {
    if (wide)
      return S == 1 ? launch_t<B200MOE_LAYOUT_Q8_0, 2, 1, 7, 2>(maps, a, st)
                    : launch_t<B200MOE_LAYOUT_Q8_0, 2, 2, 7, 2>(maps, a, st);
    return S == 1 ? launch_t<B200MOE_LAYOUT_Q8_0, 2, 1, 7, 1>(maps, a, st)
                  : launch_t<B200MOE_LAYOUT_Q8_0, 2, 2, 7, 1>(maps, a, st);
  }
  if (gate->layout == B200MOE_LAYOUT_Q8_0)
    return wide ? launch_w<B200MOE_LAYOUT_Q8_0, 2>(S, maps, a, st)
                : launch_s<B200MOE_LAYOUT_Q8_0, 2, 4, 2>(S, maps, a, st);
  if (gate->layout == B200MOE_LAYOUT_F16) return launch_s<B200MOE_LAYOUT_F16, 2, 4, 2>(S, maps, a, st);
  return wide ? launch_w<B200MOE_LAYOUT_Q4_K, 2>(S, maps, a, st)
              : launch_s<B200MOE_LAYOUT_Q4_K, 2, 4, 2>(S, maps, a, st);
}

int launch_stream_down(const void* a_in, const int32_t* seg, int pairs, int max_segment,
                       const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st) {
  if (int rc = check_weight(down, "down")) return rc;
  B200_REQUIRE(down->rows % 128 == 0,
               "stream kernel: hidden (%d) must be a multiple of 128", down->rows);
  B200_REQUIRE(ksplit >= 1 && (down->cols / KT) % ksplit == 0, "stream kernel: bad k split %d",
               ksplit);
  if (pairs == 0) return B200MOE_OK;
  int S = pick_s(max_segment);
  // max_segment is an upper bound (the token count): with top-k routing over
  // several experts a segment of 17..32 rows is rare below 33 tokens, and then
  // costs that expert a second pass; 16-token chunks keep the stage small (one
  // more stage in the ring) for everybody else.
  // The same one step up: 32-token chunks (sixteen consumer warps) for 33..64 tokens.
  if (down->experts >= 4) {
    if (S == 4) S = 2;
    else if (S == 8 && max_segment <= 64) S = 4;
  }
  CUtensorMap maps[8];
  if (int rc = weight_maps(down, &maps[0], &maps[2])) return rc;
  maps[1] = maps[0];
  maps[3] = maps[2];
  if (int rc = token_maps(maps, a_in, pairs, static_cast<uint64_t>(down->cols) * 2, S)) return rc;
  StreamArgs a{};
  a.seg = seg; a.E = down->experts; a.N = down->rows; a.K = down->cols;
  a.ntiles = down->rows / 128; a.ksplit = ksplit;
  a.stages_per_item = down->cols / KT / ksplit;
  a.P = pairs; a.act = 0; a.out_kperm = 0; a.out = d_out; a.status = device_status_ptr();
  if (down->layout == B200MOE_LAYOUT_Q8_0 && down->sub != nullptr)
    a.st0 = a.st1 = static_cast<const uint8_t*>(down->sub);
  a.total_rows = static_cast<long long>(down->experts) * down->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  const bool wide = use_wide(down->layout, S);
  if (down->layout == B200MOE_LAYOUT_Q8_0)
    return wide ? launch_w<B200MOE_LAYOUT_Q8_0, 1>(S, maps, a, st)
                : launch_s<B200MOE_LAYOUT_Q8_0, 1, 4, 2>(S, maps, a, st);
  if (down->layout == B200MOE_LAYOUT_F16) return launch_s<B200MOE_LAYOUT_F16, 1, 4, 2>(S, maps, a, st);
  return wide ? launch_w<B200MOE_LAYOUT_Q4_K, 1>(S, maps, a, st)
              : launch_s<B200MOE_LAYOUT_Q4_K, 1, 4, 2>(S, maps, a, st);
}

void set_stream_wide(int mode) { g_stream_wide = mode; }

}  // namespace b200moe
