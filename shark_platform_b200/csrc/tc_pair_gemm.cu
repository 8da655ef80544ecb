// CTA-pair variant of the tensor-core grouped expert GEMM (tcgen05, cta_group::2).
//
// STATUS: written and compile-checked only; it has not run on a GPU yet.
// Reached only with regime B200MOE_REGIME_TENSOR_PAIR (never chosen by auto).
// First run: one GPU, small shapes, compare with tc_gemm_kernel bit for bit
// (same accumulation order per output element).
//
// Why: tc_gemm_kernel (one CTA per 256 weight rows x 192 tokens) is bound by
// what one SM can ingest: per 64-k stage 16 KB of quantised weights + 24 KB of
// token tile, about 1220 clocks against 704 tensor-pipe clocks.  Here two CTAs
// of a cluster share one token tile: each loads half of its rows, the leader's
// single thread issues tcgen05.mma.cta_group::2 with M = 256 (128 weight rows
// of each CTA's own set in its own tensor memory) and N = the whole token tile,
// the hardware reads the B halves from both CTAs' shared memory.  Per SM and
// stage: 16 KB + 12 KB, and half as many MMA issues per flop.
//
// What differs from tc_gemm_kernel:
//   * cluster of 2; pair tile = (expert, two consecutive row tiles, token tile);
//     CTA rank r takes row tile 2*pt + r
//   * token slots hold <= 96 rows; both CTAs' token loads complete on the
//     LEADER's xfull barrier (cp.async.bulk.tensor ... .cta_group::2 with the
//     leader's barrier address); the leader arms it with the bytes of both halves
//   * a_ready and acc_empty live in the leader only and count the dequant
//     threads of both CTAs (remote mbarrier.arrive through mapa)
//   * xempty, a_free, acc_full exist in both CTAs and are signalled by the
//     leader's tcgen05.commit.cta_group::2 with a CTA mask of 0b11
//   * tensor memory is allocated / freed with cta_group::2 by the MMA warp of
//     BOTH CTAs (same shared-memory destination offset), freeing only after a
//     cluster-wide barrier
//   * MMA N must be a multiple of 32 (each CTA holds N/2 rows, a multiple of 16)
// No TMA load uses cluster multicast.
#include "common.cuh"
#include "kernels.h"

namespace b200moe {
namespace {

constexpr int TP_DQ_WARPS = 16;
constexpr int TP_WARP_WPROD = TP_DQ_WARPS;
constexpr int TP_WARP_XPROD = TP_DQ_WARPS + 1;
constexpr int TP_WARP_MMA = TP_DQ_WARPS + 2;
constexpr int TP_THREADS = (TP_DQ_WARPS + 3) * 32;
constexpr int TP_KT = 64;            // k per stage
constexpr int TP_ROWS = 128;         // weight rows per set and CTA
constexpr int TP_NTOK = 192;         // token rows of a pair tile / accumulator columns
constexpr int TP_NHALF = TP_NTOK / 2;
constexpr int TP_MAX_E = 64;
constexpr int TP_WSLOTS = 3;
constexpr int TP_WSET = TP_ROWS * 128;
constexpr int TP_WSLOT = 2 * TP_WSET;
constexpr int TP_XSLOTS = 8;
constexpr int TP_XSLOT = TP_NHALF * TP_KT * 2;   // 12 KB
constexpr int TP_SGROUP = 4;
constexpr int TP_SSLOTS = 2;
constexpr int TP_SSET = TP_ROWS * 32;
constexpr int TP_SSLOT = 2 * TP_SSET;
constexpr int TP_OFF_X = TP_WSLOTS * TP_WSLOT;
constexpr int TP_OFF_S = TP_OFF_X + TP_XSLOTS * TP_XSLOT;
constexpr int TP_OFF_BAR = TP_OFF_S + TP_SSLOTS * TP_SSLOT;
constexpr int TP_SMEM = 1024 + TP_OFF_BAR + 512;
constexpr uint32_t TP_COL_ACC0 = 0, TP_COL_ACC1 = 192, TP_COL_A = 384;
static_assert(TP_WSLOT % 1024 == 0 && TP_XSLOT % 1024 == 0, "slot alignment for the swizzle");
static_assert(TP_SMEM <= 232448, "shared memory budget");

struct TpArgs {
  const int32_t* seg;
  int E, N, K;
  int ntiles;      // row tiles per expert and CTA pair (N / 256 for gate+up, N / 512 for down)
  int tok_tile;    // upper bound on tokens per tile (multiple of 32, <= 192)
  int ksplit;
  int P;
  int act;
  int out_kperm;
  void* out;
  int32_t* status;
  const uint8_t* st0;
  const uint8_t* st1;
  long long total_rows;
  long long* trace;  // NULL, or [2 CTAs][TR_ROLES][TR_STAGES][TR_POINTS] clock64 stamps of CTA pair 0
};

// Diagnostic time stamps (b200moe_trace_*): the first TR_STAGES stages of the
// first CTA pair, one row per warp role.  clock64 is per SM: stamps of the two
// CTAs are not on one time base.
constexpr int TR_ROLES = 5, TR_STAGES = 256, TR_POINTS = 8;
__device__ long long g_tp_trace[2 * TR_ROLES * TR_STAGES * TR_POINTS];
bool g_tp_trace_on = false;

__device__ __forceinline__ void tr_mark(long long* trace, uint32_t rank, int role, uint32_t stage, int point) {
  if (trace != nullptr && stage < TR_STAGES)
    trace[((rank * TR_ROLES + role) * TR_STAGES + stage) * TR_POINTS + point] = clock64();
}

// ---- cluster helpers ---------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address) in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier of any CTA of the cluster (cluster-scope release)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// bounded wait on a barrier whose arrivals come from both CTAs
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag, int32_t* status) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > (1ll << 31)) {
      *abort_flag = 1;
      atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
      return false;
    }
  }
}

__device__ __forceinline__ void tp_bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Token-tile load of a CTA pair: lands in this CTA's shared memory, completes
// on `bar`, a shared::cluster address that may belong to the peer CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, int32_t x,
                                                 int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// ---- tcgen05 wrappers (cta_group::2 where the pair acts as one) ---------------
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tp_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tp_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs once all
// MMAs issued so far have completed
__device__ __forceinline__ void tp_commit_both(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor] over the CTA pair (M = 256)
__device__ __forceinline__ void tp_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tp_tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
      "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
      "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
      "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),
      "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tp_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tp_tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tp_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint64_t tp_smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1024u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ uint32_t tp_make_idesc(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <int LAYOUT, int NMAT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TP_THREADS, 1)
tc_pair_gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                    const __grid_constant__ CUtensorMap tm_s0, const __grid_constant__ CUtensorMap tm_s1,
                    const __grid_constant__ CUtensorMap tm_x16, const __grid_constant__ CUtensorMap tm_x32,
                    const __grid_constant__ CUtensorMap tm_x48, const __grid_constant__ CUtensorMap tm_x64,
                    const __grid_constant__ CUtensorMap tm_x80, const __grid_constant__ CUtensorMap tm_x96,
                    const TpArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_seg[TP_MAX_E + 1];
  __shared__ int s_prefix[TP_MAX_E + 1];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t x_base = smem_base + TP_OFF_X;
  const uint32_t scale_base = smem_base + TP_OFF_S;
  const uint32_t bar_base = smem_base + TP_OFF_BAR;
  int nb = 0;
  auto take = [&](int n) { const uint32_t b = bar_base + 8u * nb; nb += n; return b; };
  const uint32_t wfull = take(TP_WSLOTS), wempty = take(TP_WSLOTS);
  const uint32_t xfull = take(TP_XSLOTS), xempty = take(TP_XSLOTS);
  const uint32_t sfull = take(TP_SSLOTS), sempty = take(TP_SSLOTS);
  const uint32_t a_ready = take(2), a_free = take(2);
  const uint32_t acc_full_bar = take(1), acc_empty_bar = take(1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  long long* const tr = pair == 0 ? args.trace : nullptr;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < TP_WSLOTS; ++s) {
      mbar_init(wfull + 8u * s, 1);
      mbar_init(wempty + 8u * s, TP_DQ_WARPS);
    }
    for (int s = 0; s < TP_XSLOTS; ++s) {
      mbar_init(xfull + 8u * s, 1);    // used in the leader only
      mbar_init(xempty + 8u * s, 1);
    }
    for (int s = 0; s < TP_SSLOTS; ++s) {
      mbar_init(sfull + 8u * s, 1);
      mbar_init(sempty + 8u * s, TP_DQ_WARPS);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(a_ready + 8u * s, TP_DQ_WARPS);  // leader only: one arrival per warp of the filling group, both CTAs
      mbar_init(a_free + 8u * s, 1);
    }
    mbar_init(acc_full_bar, 1);
    mbar_init(acc_empty_bar, 2 * TP_DQ_WARPS);  // leader only: one arrival per dequant warp of both CTAs
    fence_mbar_init();
    int run = 0;
    for (int e = 0; e < args.E; ++e) {
      const int a = args.seg[e], b = args.seg[e + 1];
      s_seg[e] = a;
      s_prefix[e] = run;
      run += ((b - a + args.tok_tile - 1) / args.tok_tile) * args.ntiles * args.ksplit;
    }
    s_seg[args.E] = args.seg[args.E];
    s_prefix[args.E] = run;
  }
  __syncthreads();
  // the peer must be running, with its barriers initialised, before anything is
  // signalled across CTAs and before the pair allocates tensor memory together
  cluster_arrive();
  cluster_wait();
  if (warp == TP_WARP_MMA) {
    tmem_alloc2(smem_u32(&s_tmem), 512);
    tmem_relinquish2();
  }
  tp_fence_before();
  __syncthreads();
  tp_fence_after();
  const uint32_t tmem = s_tmem;
  const int total_tiles = s_prefix[args.E];
  volatile int* abort_flag = &s_abort;
  const int stages_per_tile = args.K / TP_KT / args.ksplit;  // a multiple of 4
  constexpr bool Q4 = LAYOUT == B200MOE_LAYOUT_Q4_K;
  constexpr uint32_t WSET_BYTES = Q4 ? TP_ROWS * 64 : TP_ROWS * 128;
  constexpr uint32_t SSET_BYTES = Q4 ? TP_ROWS * 32 : TP_ROWS * 16;
  // leader-side addresses of the barriers both CTAs signal
  const uint32_t xfull_leader = mapa_shared(xfull, 0);
  const uint32_t a_ready_leader = mapa_shared(a_ready, 0);
  const uint32_t acc_empty_leader = mapa_shared(acc_empty_bar, 0);

  // pair tile -> (expert, row tile of THIS CTA | k partition << 16, first token row, rows, MMA N)
  auto decode = [&](int tile, int& e, int& nt, int& row0, int& rows, int& ncols) {
    e = 0;
    while (tile >= s_prefix[e + 1]) ++e;
    const int local = tile - s_prefix[e];
    const int m = s_seg[e + 1] - s_seg[e];
    const int mtiles = (m + args.tok_tile - 1) / args.tok_tile;
    const int mt = local % mtiles;
    const int rest = local / mtiles;
    nt = (2 * (rest / args.ksplit) + static_cast<int>(rank)) | ((rest % args.ksplit) << 16);
    const int per = ((m + mtiles - 1) / mtiles + 31) & ~31;  // balanced, multiple of 32
    row0 = s_seg[e] + mt * per;
    rows = min(per, s_seg[e + 1] - row0);
    if (rows < 0) rows = 0;
    ncols = (max(rows, 1) + 31) & ~31;
  };

  if (warp == TP_WARP_WPROD) {
    // ------------------------------------------- TMA producer: weights + scales (per CTA)
    if (lane == 0) {
      uint32_t n = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        const int kbase = (nt >> 16) * stages_per_tile * TP_KT;
        nt &= 0xffff;
        const int grow0 = e * args.N + nt * (NMAT == 2 ? TP_ROWS : 2 * TP_ROWS);
        const int grow1 = NMAT == 2 ? grow0 : grow0 + TP_ROWS;
        for (int st = 0; st < stages_per_tile; st += 2, n += 2) {
          const int k0 = kbase + st * TP_KT;
          if (st % TP_SGROUP == 0) {
            const uint32_t g = n / TP_SGROUP;
            const int ss = g % TP_SSLOTS;
            if (!mbar_wait(sempty + 8u * ss, ((g / TP_SSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
            fence_proxy_async_smem();
            const uint32_t sdst = scale_base + ss * TP_SSLOT;
            const uint32_t sb = sfull + 8u * ss;
            mbar_expect_tx(sb, 2 * SSET_BYTES);
            if constexpr (Q4) {
              tma_load_2d(sdst, &tm_s0, (k0 / 32) * 4, grow0, sb);
              tma_load_2d(sdst + TP_SSET, NMAT == 2 ? &tm_s1 : &tm_s0, (k0 / 32) * 4, grow1, sb);
            } else if (args.st0 != nullptr) {
              const long long goff = static_cast<long long>(k0 / 256) * args.total_rows;
              tp_bulk_load(sdst, args.st0 + (goff + grow0) * 16, SSET_BYTES, sb);
              tp_bulk_load(sdst + TP_SSET, (NMAT == 2 ? args.st1 : args.st0) + (goff + grow1) * 16, SSET_BYTES, sb);
            } else {
              tma_load_2d(sdst, &tm_s0, (k0 / 32) * 2, grow0, sb);
              tma_load_2d(sdst + TP_SSET, NMAT == 2 ? &tm_s1 : &tm_s0, (k0 / 32) * 2, grow1, sb);
            }
          }
          const uint32_t wi = n >> 1;
          const int ws = wi % TP_WSLOTS;
          tr_mark(tr, rank, 0, n, 0);
          if (!mbar_wait(wempty + 8u * ws, ((wi / TP_WSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(tr, rank, 0, n, 1);
          fence_proxy_async_smem();
          const uint32_t wdst = smem_base + ws * TP_WSLOT;
          const uint32_t wb = wfull + 8u * ws;
          mbar_expect_tx(wb, 2 * WSET_BYTES);
          tma_load_2d(wdst, &tm_w0, Q4 ? k0 / 2 : k0, grow0, wb);
          tma_load_2d(wdst + TP_WSET, NMAT == 2 ? &tm_w1 : &tm_w0, Q4 ? k0 / 2 : k0, grow1, wb);
        }
      }
      const uint32_t wn = n >> 1;
      for (uint32_t i = wn > (uint32_t)TP_WSLOTS ? wn - TP_WSLOTS : 0; i < wn; ++i)
        mbar_wait(wfull + 8u * (i % TP_WSLOTS), (i / TP_WSLOTS) & 1u, abort_flag, args.status);
      const uint32_t gn = n / TP_SGROUP;
      for (uint32_t g = gn > (uint32_t)TP_SSLOTS ? gn - TP_SSLOTS : 0; g < gn; ++g)
        mbar_wait(sfull + 8u * (g % TP_SSLOTS), (g / TP_SSLOTS) & 1u, abort_flag, args.status);
    }
  } else if (warp == TP_WARP_XPROD) {
    // ------------------------ TMA producer: this CTA's half of the token tile
    if (lane == 0) {
      uint32_t n = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        const int half = ncols >> 1;  // multiple of 16, <= 96
        const CUtensorMap* tx = half <= 16 ? &tm_x16 : half <= 32 ? &tm_x32 : half <= 48 ? &tm_x48
                              : half <= 64 ? &tm_x64 : half <= 80 ? &tm_x80 : &tm_x96;
        const uint32_t half_bytes = static_cast<uint32_t>(half) * 128u;  // box height == half
        const int my_row0 = row0 + static_cast<int>(rank) * half;
        for (int st = 0; st < stages_per_tile; ++st, ++n) {
          const int xs = n % TP_XSLOTS;
          // freed in both CTAs by the leader's commit
          tr_mark(tr, rank, 1, n, 0);
          if (!mbar_wait(xempty + 8u * xs, ((n / TP_XSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(tr, rank, 1, n, 1);
          if (leader) mbar_expect_tx(xfull + 8u * xs, 2 * half_bytes);
          tma_load_2d_pair(x_base + xs * TP_XSLOT, tx, ((nt >> 16) * stages_per_tile + st) * TP_KT * 2,
                           my_row0, xfull_leader + 8u * xs);
        }
      }
      if (leader)
        for (uint32_t i = n > (uint32_t)TP_XSLOTS ? n - TP_XSLOTS : 0; i < n; ++i)
          mbar_wait(xfull + 8u * (i % TP_XSLOTS), (i / TP_XSLOTS) & 1u, abort_flag, args.status);
    }
  } else if (warp == TP_WARP_MMA) {
    // ------------------------------------------- MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      uint32_t n = 0, ti = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += npairs, ++ti) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        const uint32_t idesc = tp_make_idesc(256, ncols);
        if (!mbar_wait_cluster(acc_empty_bar, (ti & 1u) ^ 1u, abort_flag, args.status)) break;
        tp_fence_after();
        for (int st = 0; st < stages_per_tile; ++st, ++n) {
          const int xs = n % TP_XSLOTS;
          const int as = n & 1;
          tr_mark(tr, rank, 2, n, 0);
          if (!mbar_wait(xfull + 8u * xs, (n / TP_XSLOTS) & 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(tr, rank, 2, n, 1);
          if (!mbar_wait_cluster(a_ready + 8u * as, (n >> 1) & 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(tr, rank, 2, n, 2);
          tp_fence_after();
          const uint64_t bdesc = tp_smem_desc_sw128(x_base + xs * TP_XSLOT);
#pragma unroll
          for (int j = 0; j < TP_KT / 16; ++j) {
            const uint32_t accum = (st > 0 || j > 0) ? 1u : 0u;
            const uint64_t bd = bdesc + static_cast<uint64_t>((j * 32) >> 4);
            const uint32_t a0 = tmem + TP_COL_A + as * 64 + j * 8;
            tp_mma_ts(tmem + TP_COL_ACC0, a0, bd, idesc, accum);
            tp_mma_ts(tmem + TP_COL_ACC1, a0 + 32, bd, idesc, accum);
          }
          tp_commit_both(xempty + 8u * xs);
          tp_commit_both(a_free + 8u * as);
          tr_mark(tr, rank, 2, n, 3);
        }
        if (ok) tp_commit_both(acc_full_bar);
      }
    }
  } else {
    // ------------------------------------- dequantise (both sets) + epilogue, per CTA
    const int grp = warp >> 3;
    const int set = (warp >> 2) & 1;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const int sw = row & 7;
    uint32_t n = 0, ti = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += npairs, ++ti) {
      int e, nt, row0, rows, ncols;
      decode(tile, e, nt, row0, rows, ncols);
      for (int sg = 0; sg < stages_per_tile / TP_SGROUP && ok; ++sg) {
        const uint32_t g = n / TP_SGROUP;
        const int ss = g % TP_SSLOTS;
        if (!mbar_wait_warp(sfull + 8u * ss, (g / TP_SSLOTS) & 1u, abort_flag, args.status)) { ok = false; break; }
        uint32_t scw[8];
        if constexpr (Q4) {
          lds128(scale_base + ss * TP_SSLOT + set * TP_SSET + row * 32, *reinterpret_cast<uint32_t(*)[4]>(&scw[0]));
          lds128(scale_base + ss * TP_SSLOT + set * TP_SSET + row * 32 + 16, *reinterpret_cast<uint32_t(*)[4]>(&scw[4]));
        } else {
          lds128(scale_base + ss * TP_SSLOT + set * TP_SSET + row * 16, *reinterpret_cast<uint32_t(*)[4]>(&scw[0]));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(sempty + 8u * ss);
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4, ++n) {
          if ((s4 & 1) != grp) continue;
          const uint32_t wi = n >> 1;
          const int ws = wi % TP_WSLOTS;
          const int as = n & 1;
          long long* const trd = (wq == 0 && set == 0 && lane == 0) ? tr : nullptr;
          tr_mark(trd, rank, 3 + grp, n, 0);
          if (!mbar_wait_warp(wfull + 8u * ws, (wi / TP_WSLOTS) & 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(trd, rank, 3 + grp, n, 1);
          uint32_t v[32];
          if constexpr (Q4) {
            const uint32_t wrow = smem_base + ws * TP_WSLOT + set * TP_WSET + row * 64;
            const int sw64 = (row >> 1) & 3;
            uint32_t q[2][4];
#pragma unroll
            for (int c = 0; c < 2; ++c) lds128(wrow + (((2 * grp + c) ^ sw64) << 4), q[c]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty + 8u * ws);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint32_t sm = scw[2 * s4 + c];
              const __half2 ds = u32_as_h2(__byte_perm(sm, sm, 0x1010));
              const __half2 dm = u32_as_h2(__byte_perm(sm, sm, 0x3232));
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dequant_q4x8(q[c][j], ds, dm, *reinterpret_cast<uint32_t(*)[4]>(&v[c * 16 + j * 4]));
            }
          } else {
            const uint32_t wrow = smem_base + ws * TP_WSLOT + set * TP_WSET + row * 128;
            uint32_t q[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) lds128(wrow + (((4 * grp + c) ^ sw) << 4), q[c]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty + 8u * ws);
            const __half2 s_lo = u32_as_h2(__byte_perm(scw[s4], scw[s4], 0x1010));
            const __half2 s_hi = u32_as_h2(__byte_perm(scw[s4], scw[s4], 0x3232));
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dequant_q8x4(q[c][j], c < 2 ? s_lo : s_hi, v[c * 8 + 2 * j], v[c * 8 + 2 * j + 1]);
          }
          // this CTA's A slot is free once the pair's MMAs of stage n-2 are done
          tr_mark(trd, rank, 3 + grp, n, 2);
          if (!mbar_wait_warp(a_free + 8u * as, ((n >> 1) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          tr_mark(trd, rank, 3 + grp, n, 3);
          tp_fence_after();
          tp_tmem_st32(tmem + lane_addr + TP_COL_A + as * 64 + set * 32, v);
          tp_wait_st();
          tp_fence_before();
          tr_mark(trd, rank, 3 + grp, n, 4);
          // one arrival per warp: an arrival on the leader's barrier from the
          // peer CTA is a transaction over the SM-to-SM network
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(a_ready_leader + 8u * as);
        }
      }
      if (!ok) break;
      // ---- epilogue: this CTA's 128 rows of each set, all token columns
      if (!mbar_wait_warp(acc_full_bar, ti & 1u, abort_flag, args.status)) break;
      tp_fence_after();
      const int seg_end = row0 + rows;
      for (int c0 = (grp * 2 + set) * 16; c0 < ncols; c0 += 64) {
        uint32_t g[16], u[16];
        tp_tmem_ld16(tmem + lane_addr + TP_COL_ACC0 + c0, g);
        tp_tmem_ld16(tmem + lane_addr + TP_COL_ACC1 + c0, u);
        tp_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = row0 + c0 + j;
          if (tok >= seg_end) continue;
          if constexpr (NMAT == 2) {
            const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
            const float a = args.act == B200MOE_ACT_SILU ? silu_f(gv) : gelu_erf_f(gv);
            int col = (nt & 0xffff) * TP_ROWS + row;
            if (args.out_kperm) col = (col & ~7) | ((col & 3) << 1) | ((col >> 2) & 1);
            static_cast<__half*>(args.out)[static_cast<size_t>(tok) * args.N + col] = to_half_sat(a * uv, args.status);
          } else {
            float* o = static_cast<float*>(args.out) +
                       static_cast<size_t>(nt >> 16) * args.P * args.N +
                       static_cast<size_t>(tok) * args.N + (nt & 0xffff) * (2 * TP_ROWS) + row;
            o[0] = __uint_as_float(g[j]);
            o[TP_ROWS] = __uint_as_float(u[j]);
          }
        }
      }
      tp_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
    }
  }

  // ---- teardown: both CTAs are done with tensor memory, shared memory and
  // each other's barriers before either frees or leaves
  tp_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == TP_WARP_MMA) {
    tp_fence_after();
    tmem_dealloc2(tmem, 512);
  }
}

template <int LAYOUT, int NMAT>
int tp_launch(const CUtensorMap* maps, const TpArgs& a_in, cudaStream_t st) {
  auto kern = tc_pair_gemm_kernel<LAYOUT, NMAT>;
  TpArgs a = a_in;
  a.trace = nullptr;
  if (g_tp_trace_on) {
    void* p = nullptr;
    B200_CHECK_CUDA(cudaGetSymbolAddress(&p, g_tp_trace));
    B200_CHECK_CUDA(cudaMemsetAsync(p, 0, sizeof(long long) * 2 * TR_ROLES * TR_STAGES * TR_POINTS, st));
    a.trace = static_cast<long long*>(p);
  }
  static bool configured[16] = {};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM));
    configured[dev] = true;
  }
  // cluster dimensions are compiled into the kernel; the grid must be even
  const int ctas = sm_count() & ~1;
  kern<<<ctas, TP_THREADS, TP_SMEM, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                                          maps[6], maps[7], maps[8], maps[9], a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// Half-tile token maps with box heights 16 .. 96 in steps of 16 (maps[4..9]).
int tp_token_maps(CUtensorMap* maps, const void* x, int pairs, uint64_t row_bytes) {
  for (int i = 0; i < 6; ++i)
    if (int rc = make_tmap_2d_sw(&maps[4 + i], x, pairs, row_bytes, 16 * (i + 1), 128, 128)) return rc;
  return B200MOE_OK;
}

int tp_weight_map(const b200moe_weight_t* w, CUtensorMap* tw, CUtensorMap* ts) {
  const uint64_t rows = static_cast<uint64_t>(w->experts) * w->rows;
  if (w->layout == B200MOE_LAYOUT_Q4_K) {
    if (int rc = make_tmap_2d_sw(tw, w->qs, rows, w->cols / 2, TP_ROWS, 64, 64)) return rc;
    return make_tmap_2d_sw(ts, w->sub, rows, static_cast<uint64_t>(w->cols) / 32 * 4, TP_ROWS, 32, 0);
  }
  if (int rc = make_tmap_2d_sw(tw, w->qs, rows, w->cols, TP_ROWS, 128, 128)) return rc;
  return make_tmap_2d_sw(ts, w->d, rows, static_cast<uint64_t>(w->cols) / 32 * 2, TP_ROWS, 16, 0);
}

}  // namespace

int pair_trace_enable(bool on) {
  g_tp_trace_on = on;
  return B200MOE_OK;
}

int pair_trace_read(long long* out, size_t count) {
  const size_t n = static_cast<size_t>(2) * TR_ROLES * TR_STAGES * TR_POINTS;
  B200_REQUIRE(out != nullptr && count >= n, "trace_read: the buffer must hold %zu values", n);
  B200_CHECK_CUDA(cudaDeviceSynchronize());
  B200_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_tp_trace, sizeof(long long) * n));
  return B200MOE_OK;
}

// The pair kernel needs an even number of row tiles per expert.
bool tc_pair_supported_gate_up(const b200moe_weight_t* gate) {
  return (gate->layout == B200MOE_LAYOUT_Q8_0 || gate->layout == B200MOE_LAYOUT_Q4_K) &&
         gate->cols % 256 == 0 && gate->rows % (2 * TP_ROWS) == 0;
}
bool tc_pair_supported_down(const b200moe_weight_t* down) {
  return (down->layout == B200MOE_LAYOUT_Q8_0 || down->layout == B200MOE_LAYOUT_Q4_K) &&
         down->cols % 256 == 0 && down->rows % (4 * TP_ROWS) == 0;
}

int launch_tc_pair_gate_up(const void* xs, const int32_t* seg, int pairs, int tok_tile,
                           const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                           int out_kperm, void* a_out, cudaStream_t st) {
  B200_REQUIRE(tc_pair_supported_gate_up(gate) && tc_pair_supported_gate_up(up),
               "pair kernel: gate/up layout or shape unsupported");
  B200_REQUIRE(gate->rows == up->rows && gate->cols == up->cols && gate->experts == up->experts &&
                   gate->layout == up->layout,
               "pair kernel: gate and up shapes or layouts differ");
  B200_REQUIRE(tok_tile % 32 == 0 && tok_tile >= 32 && tok_tile <= TP_NTOK, "pair kernel: bad token tile %d", tok_tile);
  if (pairs == 0) return B200MOE_OK;
  CUtensorMap maps[10];
  if (int rc = tp_weight_map(gate, &maps[0], &maps[2])) return rc;
  if (int rc = tp_weight_map(up, &maps[1], &maps[3])) return rc;
  if (int rc = tp_token_maps(maps, xs, pairs, static_cast<uint64_t>(gate->cols) * 2)) return rc;
  TpArgs a{};
  a.seg = seg; a.E = gate->experts; a.N = gate->rows; a.K = gate->cols;
  a.ntiles = gate->rows / (2 * TP_ROWS); a.tok_tile = tok_tile; a.P = pairs; a.act = act;
  a.ksplit = 1;
  a.out_kperm = out_kperm;
  a.out = a_out; a.status = device_status_ptr();
  a.total_rows = static_cast<long long>(gate->experts) * gate->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  if (gate->layout == B200MOE_LAYOUT_Q4_K) return tp_launch<B200MOE_LAYOUT_Q4_K, 2>(maps, a, st);
  if (gate->sub != nullptr && up->sub != nullptr) {
    a.st0 = static_cast<const uint8_t*>(gate->sub);
    a.st1 = static_cast<const uint8_t*>(up->sub);
  }
  return tp_launch<B200MOE_LAYOUT_Q8_0, 2>(maps, a, st);
}

int launch_tc_pair_down(const void* a_in, const int32_t* seg, int pairs, int tok_tile,
                        const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st) {
  B200_REQUIRE(tc_pair_supported_down(down), "pair kernel: down layout or shape unsupported");
  B200_REQUIRE(tok_tile % 32 == 0 && tok_tile >= 32 && tok_tile <= TP_NTOK, "pair kernel: bad token tile %d", tok_tile);
  B200_REQUIRE(ksplit >= 1 && (down->cols / TP_KT) % (4 * ksplit) == 0, "pair kernel: bad k split %d", ksplit);
  if (pairs == 0) return B200MOE_OK;
  CUtensorMap maps[10];
  if (int rc = tp_weight_map(down, &maps[0], &maps[2])) return rc;
  maps[1] = maps[0];
  maps[3] = maps[2];
  if (int rc = tp_token_maps(maps, a_in, pairs, static_cast<uint64_t>(down->cols) * 2)) return rc;
  TpArgs a{};
  a.seg = seg; a.E = down->experts; a.N = down->rows; a.K = down->cols;
  a.ntiles = down->rows / (4 * TP_ROWS); a.tok_tile = tok_tile; a.P = pairs; a.act = 0;
  a.ksplit = ksplit;
  a.out = d_out; a.status = device_status_ptr();
  a.total_rows = static_cast<long long>(down->experts) * down->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  if (down->layout == B200MOE_LAYOUT_Q4_K) return tp_launch<B200MOE_LAYOUT_Q4_K, 1>(maps, a, st);
  if (down->sub != nullptr) a.st0 = a.st1 = static_cast<const uint8_t*>(down->sub);
  return tp_launch<B200MOE_LAYOUT_Q8_0, 1>(maps, a, st);
}

}  // namespace b200moe
