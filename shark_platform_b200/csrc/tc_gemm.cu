// Tensor-core grouped expert GEMM for the prefill regime (many tokens per
// expert): tcgen05.mma with fp32 accumulators in tensor memory.
//
// Orientation is "swap-AB" with the A operand in tensor memory: a tile of 128
// weight rows is M, up to 192 tokens of one expert are N.  Weights never touch
// shared memory in dequantised form: warps read the TMA-staged quantised bytes
// (one thread per weight row), dequantise to fp16 in registers and write the
// row into tensor memory with tcgen05.st, where it is the A operand of the next
// MMAs.  The token rows (fp16, K-major, 128-byte swizzle) are the B operand, read
// from shared memory through a matrix descriptor.  Shared memory therefore only
// carries quantised bytes and token tiles.
//
// A CTA holds two row sets per tile, each with its own accumulator:
// gate rows + up rows of the same 128 columns (SiLU/GELU-gated product in the
// epilogue), or 256 consecutive rows of the down matrix.
//
// Three independent shared-memory rings, because their slots live for very
// different times:
//   weights  2 slots x (2 sets x 128 rows x 128 k) int8, 128-byte swizzle;
//            a slot is free again as soon as the dequant warps have read it
//   tokens   6 slots x (192 rows x 64 k) fp16; a slot is held until the MMAs
//            that read it have completed
//   scales   2 slots x (2 sets x 128 rows x 8) fp16 = 256 k
//
// Warp roles (608 threads, one CTA per SM, persistent over tiles):
//   warps 0-7   group 0: dequantise the even 64-k stages (warps 0-3 set 0,
//               warps 4-7 set 1; warp w owns TMEM lanes 32(w%4)..+31), epilogue
//   warps 8-15  group 1: the same for the odd stages, so that one group's
//               tensor-memory store latency hides behind the other's arithmetic
//   warp  16    TMA producer for weights and scales
//   warp  17    TMA producer for token tiles
//   warp  18    TMEM allocation; one lane issues the MMAs of row set 0 and commits
//   warp  19    one lane issues the MMAs of row set 1
// Two issuers because issuing is what the loop is short of: an MMA costs its
// issuing thread ~70 clocks, eight per 64-k stage plus the barrier waits exceed
// the 768 clocks the tensor pipe needs for them, so with one issuer the pipe runs
// dry every stage.  Each row set has its own A-slot barriers, so the two sets
// are independent pipelines that share only the token tiles.
//
// Tensor-memory columns (512 allocated): accumulators at 0 and 192 (192 fp32
// columns each), two A staging slots of 2 x 32 columns at 384..511.
//
// All mbarrier waits are bounded; on expiry the CTA raises its abort flag, every
// role falls out of its loops, the CTA frees its tensor memory and returns.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int TC_DQ_WARPS = 16;
constexpr int TC_WARP_WPROD = TC_DQ_WARPS;
constexpr int TC_WARP_XPROD = TC_DQ_WARPS + 1;
constexpr int TC_WARP_MMA = TC_DQ_WARPS + 2;   // issues the MMAs of row set 0 (and owns the TMEM allocation)
constexpr int TC_WARP_MMA1 = TC_DQ_WARPS + 3;  // issues the MMAs of row set 1
constexpr int TC_THREADS = (TC_DQ_WARPS + 4) * 32;
constexpr int TC_KT = 64;            // k per stage (one token slot, one A slot)
constexpr int TC_ROWS = 128;         // weight rows per set
constexpr int TC_NTOK = 192;         // largest token tile / accumulator width
constexpr int TC_MAX_E = 64;
constexpr int TC_WSET = TC_ROWS * 128;          // bytes of one set in a weight slot (128 k)
constexpr int TC_WSLOT = 2 * TC_WSET;
constexpr int TC_SGROUP = 4;                    // stages covered by one scale tile (256 k)
constexpr int TC_SSLOTS = 2;
constexpr int TC_SSET = TC_ROWS * 32;           // per row and group: 8 fp16 scales (Q8_0, 16 B used) or 8 half2 scale/min pairs (Q4_K)
constexpr int TC_SSLOT = 2 * TC_SSET;

// Geometry for token tiles of at most NMAX rows.  The two accumulators take
// 2 x NMAX tensor-memory columns; what is left of the 512 holds A staging slots
// of 64 columns, so narrow tiles get a deeper A ring (the MMA lane and the
// dequant warps then rarely wait for each other) and, because their token slots
// are small, a deeper weight ring (more bytes in flight per SM, which is what a
// weight-streaming tile needs).
template <int NMAX>
struct TcCfg {
  static_assert(NMAX == 64 || NMAX == 128 || NMAX == 192, "token tile widths: 64, 128, 192");
  static constexpr int ASLOTS = (512 - 2 * NMAX) / 64;  // 6, 4, 2 (even: a slot belongs to one dequant group)
  static constexpr int WSLOTS = NMAX == 192 ? 2 : NMAX == 128 ? 3 : 5;
  // a token slot holds two 64-k stages (two swizzled sub-tiles of NMAX rows x 128 B):
  // one wait and one release per 128 k on the issuing lanes, whose instruction
  // stream is the kernel's critical path
  static constexpr int XSLOTS = 3;
  static constexpr int XSUB = NMAX * TC_KT * 2;
  static constexpr int XSLOT = 2 * XSUB;
  static constexpr int OFF_X = WSLOTS * TC_WSLOT;
  static constexpr int OFF_S = OFF_X + XSLOTS * XSLOT;
  static constexpr int OFF_BAR = OFF_S + TC_SSLOTS * TC_SSLOT;
  static constexpr int SMEM = 1024 + OFF_BAR + 512;
  static constexpr uint32_t COL_ACC0 = 0, COL_ACC1 = NMAX, COL_A = 2 * NMAX;
  static_assert(XSLOT % 1024 == 0 && TC_WSLOT % 1024 == 0, "slot alignment for the swizzle");
  static_assert(SMEM <= 232448, "shared memory budget");
  static_assert(2 * (WSLOTS + XSLOTS + TC_SSLOTS + 2 * ASLOTS) + 2 <= 64, "barrier area");
};

struct TcArgs {
  const int32_t* seg;
  int E, N, K;
  int ntiles;      // row tiles per expert (N / 128 for gate+up, N / 256 for down)
  int tok_tile;    // upper bound on tokens per tile (multiple of 16, <= 192)
  int ksplit;      // k partitions per tile (down only); partial kc goes to out + kc*P*N
  int P;
  int act;
  int out_kperm;   // gate/up only: interleave output columns for a Q4_K down matrix
  void* out;
  int32_t* status;
  // scales transposed to [K/256][rows][8] (one contiguous run per row tile and
  // 256-k group) or NULL = fetch them from `d` as 16-byte TMA rows
  const uint8_t* st0;
  const uint8_t* st1;
  long long total_rows;
};

__device__ __forceinline__ void tc_bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// ---- tcgen05 wrappers ------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The four K=16 MMAs of a 64-k stage in one statement: A at a_tmem + 8 j columns,
// B descriptors differing in the start-address field only (32 bytes = 2 units
// per K step; the upper descriptor word is constant).  The first one overwrites
// the accumulator when `accumulate` is 0.
__device__ __forceinline__ void tc_mma_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo,
                                             uint32_t b_desc_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 d0, d1, d2, d3;\n\t.reg .b32 l1, l2, l3, a1, a2, a3;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.ne.b32 t, %4, 0;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "mov.b64 d0, {%2, %3};\n\tmov.b64 d1, {l1, %3};\n\tmov.b64 d2, {l2, %3};\n\tmov.b64 d3, {l3, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d0, %4, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %4, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], d2, %4, t;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], d3, %4, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
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
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of
// 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);          // start address
  d |= static_cast<uint64_t>(1024u >> 4) << 32;                // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                         // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B
  return d;
}

// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major.
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

template <int LAYOUT, int NMAT, int NMAX>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
               const __grid_constant__ CUtensorMap tm_s0, const __grid_constant__ CUtensorMap tm_s1,
               const __grid_constant__ CUtensorMap tm_x16, const __grid_constant__ CUtensorMap tm_x32,
               const __grid_constant__ CUtensorMap tm_x64, const __grid_constant__ CUtensorMap tm_x96,
               const __grid_constant__ CUtensorMap tm_x128, const __grid_constant__ CUtensorMap tm_x192,
               const TcArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_seg[TC_MAX_E + 1];
  __shared__ int s_prefix[TC_MAX_E + 1];
  __shared__ int s_abort;
  __shared__ uint32_t s_tmem;

  using G = TcCfg<NMAX>;
  constexpr int TC_WSLOTS = G::WSLOTS, TC_XSLOTS = G::XSLOTS, TC_XSLOT = G::XSLOT, TC_XSUB = G::XSUB, TC_ASLOTS = G::ASLOTS;
  constexpr uint32_t TC_COL_ACC0 = G::COL_ACC0, TC_COL_ACC1 = G::COL_ACC1, TC_COL_A = G::COL_A;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t x_base = smem_base + G::OFF_X;
  const uint32_t scale_base = smem_base + G::OFF_S;
  const uint32_t bar_base = smem_base + G::OFF_BAR;
  int nb = 0;
  auto take = [&](int n) { const uint32_t b = bar_base + 8u * nb; nb += n; return b; };
  const uint32_t wfull = take(TC_WSLOTS), wempty = take(TC_WSLOTS);
  const uint32_t xfull = take(TC_XSLOTS), xempty = take(TC_XSLOTS);
  const uint32_t sfull = take(TC_SSLOTS), sempty = take(TC_SSLOTS);
  const uint32_t a_ready = take(2 * TC_ASLOTS), a_free = take(2 * TC_ASLOTS);  // [slot][row set]
  const uint32_t acc_full_bar = take(1), acc_empty_bar = take(1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < TC_WSLOTS; ++s) {
      mbar_init(wfull + 8u * s, 1);
      mbar_init(wempty + 8u * s, TC_DQ_WARPS);
    }
    for (int s = 0; s < TC_XSLOTS; ++s) {
      mbar_init(xfull + 8u * s, 1);
      mbar_init(xempty + 8u * s, 2);  // both issuers commit
    }
    for (int s = 0; s < TC_SSLOTS; ++s) {
      mbar_init(sfull + 8u * s, 1);
      mbar_init(sempty + 8u * s, TC_DQ_WARPS);
    }
    for (int s = 0; s < 2 * TC_ASLOTS; ++s) {
      mbar_init(a_ready + 8u * s, TC_DQ_WARPS / 4);  // one arrival per warp of the group and row set that fills it
      mbar_init(a_free + 8u * s, 1);
    }
    mbar_init(acc_full_bar, 2);  // both issuers commit
    mbar_init(acc_empty_bar, TC_DQ_WARPS);  // one arrival per dequant warp
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
  if (warp == TC_WARP_MMA) {
    tmem_alloc(smem_u32(&s_tmem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  const int total_tiles = s_prefix[args.E];
  volatile int* abort_flag = &s_abort;
  const int stages_per_tile = args.K / TC_KT / args.ksplit;  // a multiple of 4
  constexpr bool Q4 = LAYOUT == B200MOE_LAYOUT_Q4_K;
  constexpr uint32_t WSET_BYTES = Q4 ? TC_ROWS * 64 : TC_ROWS * 128;  // one set, 128 k
  constexpr uint32_t SSET_BYTES = Q4 ? TC_ROWS * 32 : TC_ROWS * 16;   // one set, 256 k

  // tile -> (expert, row tile | k partition << 16, first token row, token rows, MMA N)
  auto decode = [&](int tile, int& e, int& nt, int& row0, int& rows, int& ncols) {
    e = 0;
    while (tile >= s_prefix[e + 1]) ++e;
    const int local = tile - s_prefix[e];
    const int m = s_seg[e + 1] - s_seg[e];
    const int mtiles = (m + args.tok_tile - 1) / args.tok_tile;
    const int mt = local % mtiles;
    const int rest = local / mtiles;
    nt = (rest / args.ksplit) | ((rest % args.ksplit) << 16);
    const int per = ((m + mtiles - 1) / mtiles + 15) & ~15;  // balanced, multiple of 16
    row0 = s_seg[e] + mt * per;
    rows = min(per, s_seg[e + 1] - row0);
    if (rows < 0) rows = 0;
    ncols = (max(rows, 1) + 15) & ~15;
  };

  if (warp == TC_WARP_WPROD) {
    // ------------------------------------------- TMA producer: weights + scales
    if (lane == 0) {
      uint32_t n = 0;  // global stage counter; weight slots advance every 2, scale slots every 4
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        const int kbase = (nt >> 16) * stages_per_tile * TC_KT;
        nt &= 0xffff;
        const int grow0 = e * args.N + nt * (NMAT == 2 ? TC_ROWS : 2 * TC_ROWS);
        const int grow1 = NMAT == 2 ? grow0 : grow0 + TC_ROWS;
        for (int st = 0; st < stages_per_tile; st += 2, n += 2) {
          const int k0 = kbase + st * TC_KT;
          if (st % TC_SGROUP == 0) {
            const uint32_t g = n / TC_SGROUP;
            const int ss = g % TC_SSLOTS;
            if (!mbar_wait(sempty + 8u * ss, ((g / TC_SSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
            fence_proxy_async_smem();
            const uint32_t sdst = scale_base + ss * TC_SSLOT;
            const uint32_t sb = sfull + 8u * ss;
            mbar_expect_tx(sb, 2 * SSET_BYTES);
            if constexpr (Q4) {
              tma_load_2d(sdst, &tm_s0, (k0 / 32) * 4, grow0, sb);
              tma_load_2d(sdst + TC_SSET, NMAT == 2 ? &tm_s1 : &tm_s0, (k0 / 32) * 4, grow1, sb);
            } else if (args.st0 != nullptr) {
              const long long goff = static_cast<long long>(k0 / 256) * args.total_rows;
              tc_bulk_load(sdst, args.st0 + (goff + grow0) * 16, SSET_BYTES, sb);
              tc_bulk_load(sdst + TC_SSET, (NMAT == 2 ? args.st1 : args.st0) + (goff + grow1) * 16, SSET_BYTES, sb);
            } else {
              tma_load_2d(sdst, &tm_s0, (k0 / 32) * 2, grow0, sb);
              tma_load_2d(sdst + TC_SSET, NMAT == 2 ? &tm_s1 : &tm_s0, (k0 / 32) * 2, grow1, sb);
            }
          }
          const uint32_t wi = n >> 1;
          const int ws = wi % TC_WSLOTS;
          if (!mbar_wait(wempty + 8u * ws, ((wi / TC_WSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          fence_proxy_async_smem();
          const uint32_t wdst = smem_base + ws * TC_WSLOT;
          const uint32_t wb = wfull + 8u * ws;
          mbar_expect_tx(wb, 2 * WSET_BYTES);
          tma_load_2d(wdst, &tm_w0, Q4 ? k0 / 2 : k0, grow0, wb);
          tma_load_2d(wdst + TC_WSET, NMAT == 2 ? &tm_w1 : &tm_w0, Q4 ? k0 / 2 : k0, grow1, wb);
        }
      }
      // do not leave while copies may still land in this CTA's shared memory
      const uint32_t wn = n >> 1;
      for (uint32_t i = wn > (uint32_t)TC_WSLOTS ? wn - TC_WSLOTS : 0; i < wn; ++i)
        mbar_wait(wfull + 8u * (i % TC_WSLOTS), (i / TC_WSLOTS) & 1u, abort_flag, args.status);
      const uint32_t gn = n / TC_SGROUP;
      for (uint32_t g = gn > (uint32_t)TC_SSLOTS ? gn - TC_SSLOTS : 0; g < gn; ++g)
        mbar_wait(sfull + 8u * (g % TC_SSLOTS), (g / TC_SSLOTS) & 1u, abort_flag, args.status);
    }
  } else if (warp == TC_WARP_XPROD) {
    // -------------------------------------------------- TMA producer: token tiles
    if (lane == 0) {
      uint32_t n = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        // the per-SM TMA rate is one 128-byte box row per few clocks, whether or
        // not the row is used: take the shortest box that covers the tile
        const CUtensorMap* tx = ncols <= 16 ? &tm_x16 : ncols <= 32 ? &tm_x32 : ncols <= 64 ? &tm_x64
                              : ncols <= 96 ? &tm_x96 : ncols <= 128 ? &tm_x128 : &tm_x192;
        const uint32_t xbytes = (ncols <= 16 ? 16 : ncols <= 32 ? 32 : ncols <= 64 ? 64
                               : ncols <= 96 ? 96 : ncols <= 128 ? 128 : 192) * 128;
        for (int st = 0; st < stages_per_tile; st += 2, ++n) {  // n counts slots = pairs of stages
          const int xs = n % TC_XSLOTS;
          if (!mbar_wait(xempty + 8u * xs, ((n / TC_XSLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          const uint32_t xb = xfull + 8u * xs;
          const int x0 = ((nt >> 16) * stages_per_tile + st) * TC_KT * 2;
          mbar_expect_tx(xb, 2 * xbytes);
          tma_load_2d(x_base + xs * TC_XSLOT, tx, x0, row0, xb);
          tma_load_2d(x_base + xs * TC_XSLOT + TC_XSUB, tx, x0 + TC_KT * 2, row0, xb);
        }
      }
      for (uint32_t i = n > (uint32_t)TC_XSLOTS ? n - TC_XSLOTS : 0; i < n; ++i)
        mbar_wait(xfull + 8u * (i % TC_XSLOTS), (i / TC_XSLOTS) & 1u, abort_flag, args.status);
    }
  } else if (warp == TC_WARP_MMA || warp == TC_WARP_MMA1) {
    // ------------------------------------------ MMA issuers, one per row set
    if (lane == 0) {
      const int mset = warp - TC_WARP_MMA;
      const uint32_t acc = tmem + (mset == 0 ? TC_COL_ACC0 : TC_COL_ACC1);
      uint32_t ti = 0;
      bool ok = true;
      // slot indices and phase parities advance by counters: this lane's
      // instruction stream is the kernel's critical path (every instruction of
      // it was measured at 15-20 clocks beside the sixteen dequantising warps)
      uint32_t xs = 0, xph = 0, as = 0, aph = 0;
      static_assert(TC_KT == 64, "tc_mma_ts_x4 issues the four K steps of a 64-k stage");
      const uint32_t desc_hi = static_cast<uint32_t>(smem_desc_sw128(0) >> 32);
      const uint32_t a_set = tmem + TC_COL_A + mset * 32;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++ti) {
        int e, nt, row0, rows, ncols;
        decode(tile, e, nt, row0, rows, ncols);
        const uint32_t idesc = make_idesc(128, ncols);
        if (!mbar_wait(acc_empty_bar, (ti & 1u) ^ 1u, abort_flag, args.status)) break;
        tc_fence_after();
        for (int st = 0; st < stages_per_tile; ++st) {
          const uint32_t ab = 8u * (2 * as + mset);
          const uint32_t sub = static_cast<uint32_t>(st) & 1u;  // half of the token slot (tiles hold an even number of stages)
          if ((sub == 0 && !mbar_wait(xfull + 8u * xs, xph, abort_flag, args.status)) ||
              !mbar_wait(a_ready + ab, aph, abort_flag, args.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t b_lo = ((x_base + xs * TC_XSLOT + sub * TC_XSUB) & 0x3FFFFu) >> 4;
          tc_mma_ts_x4(acc, a_set + as * 64, b_lo, desc_hi, idesc, st > 0 ? 1u : 0u);
          tc_commit(a_free + ab);
          if (sub) {
            tc_commit(xempty + 8u * xs);
            if (++xs == TC_XSLOTS) { xs = 0; xph ^= 1u; }
          }
          if (++as == TC_ASLOTS) { as = 0; aph ^= 1u; }
        }
        if (ok) tc_commit(acc_full_bar);
      }
    }
  } else {
    // ------------------------------------- dequantise (both sets) + epilogue
    const int grp = warp >> 3;              // stage parity this warp works on
    const int set = (warp >> 2) & 1;        // row set: 0 or 1
    const int wq = warp & 3;                // TMEM lane quarter
    const int row = wq * 32 + lane;         // weight row within the set = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const int sw = row & 7;                 // 128-byte swizzle term of this row
    uint32_t n = 0, ti = 0;
    bool ok = true;

    // Drains the two accumulators of a finished tile.  Each of the four
    // (group, set) warp sets takes every fourth 16-token column chunk.
    auto epilogue = [&](int nt, int row0, int rows, int ncols, uint32_t tix) -> bool {
      if (!mbar_wait_warp(acc_full_bar, tix & 1u, abort_flag, args.status)) return false;
      tc_fence_after();
      if constexpr (NMAT == 2) {
        int col = (nt & 0xffff) * TC_ROWS + row;
        if (args.out_kperm) col = (col & ~7) | ((col & 3) << 1) | ((col >> 2) & 1);
        __half* obase = static_cast<__half*>(args.out) + static_cast<size_t>(row0) * args.N + col;
        const size_t ostride = static_cast<size_t>(args.N);
        const bool silu = args.act == B200MOE_ACT_SILU;
        float amax = 0.f;
        for (int c0 = (grp * 2 + set) * 16; c0 < ncols; c0 += 64) {
#pragma unroll 1
          for (int h8 = 0; h8 < 16; h8 += 8) {
            uint32_t g[8], u[8];
            tmem_ld8(tmem + lane_addr + TC_COL_ACC0 + c0 + h8, g);
            tmem_ld8(tmem + lane_addr + TC_COL_ACC1 + c0 + h8, u);
            tmem_wait_ld();
            __half* o = obase + static_cast<size_t>(c0 + h8) * ostride;
            const int lim = rows - c0 - h8;  // token rows of the segment among these eight
            if (lim >= 8) {
              if (silu) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float v = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
                  amax = fmaxf(amax, fabsf(v));
                  o[j * ostride] = to_half_sat(v);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float v = gelu_erf_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
                  amax = fmaxf(amax, fabsf(v));
                  o[j * ostride] = to_half_sat(v);
                }
              }
            } else {
              // columns past the segment are products with another expert's
              // token rows: neither stored nor range-checked
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (j < lim) {
                  const float gv = __uint_as_float(g[j]);
                  const float v = (silu ? silu_f(gv) : gelu_erf_f(gv)) * __uint_as_float(u[j]);
                  amax = fmaxf(amax, fabsf(v));
                  o[j * ostride] = to_half_sat(v);
                }
              }
            }
          }
        }
        if (amax >= 65520.0f) atomicOr(args.status, DEV_WARN_SATURATED);
      } else {
        float* obase = static_cast<float*>(args.out) + static_cast<size_t>(nt >> 16) * args.P * args.N +
                       static_cast<size_t>(row0) * args.N + (nt & 0xffff) * (2 * TC_ROWS) + row;
        const size_t ostride = static_cast<size_t>(args.N);
        for (int c0 = (grp * 2 + set) * 16; c0 < ncols; c0 += 64) {
          uint32_t g[16], u[16];
          tmem_ld16(tmem + lane_addr + TC_COL_ACC0 + c0, g);
          tmem_ld16(tmem + lane_addr + TC_COL_ACC1 + c0, u);
          tmem_wait_ld();
          float* o = obase + static_cast<size_t>(c0) * ostride;
          const int lim = rows - c0;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < lim) {
              o[j * ostride] = __uint_as_float(g[j]);
              o[j * ostride + TC_ROWS] = __uint_as_float(u[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar);
      return true;
    };

    // The epilogue of tile t runs after this warp has handed the first stage of
    // tile t+1 to its issuer (the A ring gives each group one slot, so exactly
    // one stage can be staged ahead): the wait for tile t's last MMAs and the
    // restart of the pipeline overlap.
    bool have_prev = false;
    int p_nt = 0, p_row0 = 0, p_rows = 0, p_ncols = 0;
    uint32_t p_ti = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++ti) {
      int e, nt, row0, rows, ncols;
      decode(tile, e, nt, row0, rows, ncols);
      for (int sg = 0; sg < stages_per_tile / TC_SGROUP && ok; ++sg) {
        const uint32_t g = n / TC_SGROUP;
        const int ss = g % TC_SSLOTS;
        if (!mbar_wait_warp(sfull + 8u * ss, (g / TC_SSLOTS) & 1u, abort_flag, args.status)) { ok = false; break; }
        // Q8_0: 8 fp16 block scales of the 256-k group; Q4_K: 8 (scale, min) half2 pairs
        uint32_t scw[8];
        if constexpr (Q4) {
          lds128(scale_base + ss * TC_SSLOT + set * TC_SSET + row * 32, *reinterpret_cast<uint32_t(*)[4]>(&scw[0]));
          lds128(scale_base + ss * TC_SSLOT + set * TC_SSET + row * 32 + 16, *reinterpret_cast<uint32_t(*)[4]>(&scw[4]));
        } else {
          lds128(scale_base + ss * TC_SSLOT + set * TC_SSET + row * 16, *reinterpret_cast<uint32_t(*)[4]>(&scw[0]));
        }
        fence_proxy_async_smem();  // reads done before TMA may refill the slot
        __syncwarp();
        if (lane == 0) mbar_arrive(sempty + 8u * ss);
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4, ++n) {
          if ((s4 & 1) != grp) continue;
          // this group's half (64 k) of the weight slot
          const uint32_t wi = n >> 1;
          const int ws = wi % TC_WSLOTS;
          const int as = n % TC_ASLOTS;  // even slot count: slot parity == this group's stage parity
          if (!mbar_wait_warp(wfull + 8u * ws, (wi / TC_WSLOTS) & 1u, abort_flag, args.status)) { ok = false; break; }
          uint32_t v[32];
          if constexpr (Q4) {
            // 64-byte rows (128 k of nibbles), 64-byte swizzle; this stage = chunks 2*grp, 2*grp+1
            const uint32_t wrow = smem_base + ws * TC_WSLOT + set * TC_WSET + row * 64;
            const int sw64 = (row >> 1) & 3;
            uint32_t q[2][4];
#pragma unroll
            for (int c = 0; c < 2; ++c) lds128(wrow + (((2 * grp + c) ^ sw64) << 4), q[c]);
            fence_proxy_async_smem();  // reads done before TMA may refill the slot
            __syncwarp();
            if (lane == 0) mbar_arrive(wempty + 8u * ws);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint32_t sm = scw[2 * s4 + c];  // sub-block (32 k) scale / min
              const __half2 ds = u32_as_h2(__byte_perm(sm, sm, 0x1010));
              const __half2 dm = u32_as_h2(__byte_perm(sm, sm, 0x3232));
#pragma unroll
              for (int j = 0; j < 4; ++j)
                dequant_q4x8(q[c][j], ds, dm, *reinterpret_cast<uint32_t(*)[4]>(&v[c * 16 + j * 4]));
            }
          } else {
            const uint32_t wrow = smem_base + ws * TC_WSLOT + set * TC_WSET + row * 128;
            uint32_t q[4][4];
#pragma unroll
            for (int c = 0; c < 4; ++c) lds128(wrow + (((4 * grp + c) ^ sw) << 4), q[c]);
            fence_proxy_async_smem();  // reads done before TMA may refill the slot
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
          if (!mbar_wait_warp(a_free + 8u * (2 * as + set), ((n / TC_ASLOTS) & 1u) ^ 1u, abort_flag, args.status)) { ok = false; break; }
          tc_fence_after();
          tmem_st32(tmem + lane_addr + TC_COL_A + as * 64 + set * 32, v);
          tmem_wait_st();
          tc_fence_before();
          // one arrival per warp: 256 arrivals per stage on one barrier word
          // serialise in shared memory
          __syncwarp();
          if (lane == 0) mbar_arrive(a_ready + 8u * (2 * as + set));
          if (s4 < 2 && sg == 0 && have_prev) {
            have_prev = false;
            if (!epilogue(p_nt, p_row0, p_rows, p_ncols, p_ti)) { ok = false; break; }
          }
        }
      }
      if (!ok) break;
      have_prev = true;
      p_nt = nt; p_row0 = row0; p_rows = rows; p_ncols = ncols; p_ti = ti;
    }
    if (ok && have_prev) epilogue(p_nt, p_row0, p_rows, p_ncols, p_ti);
  }


  // ---- teardown: everyone is done with tensor memory before it is freed
  tc_fence_before();
  __syncthreads();
  if (warp == TC_WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int LAYOUT, int NMAT, int NMAX>
int tc_launch_n(const CUtensorMap* maps, const TcArgs& a, cudaStream_t st) {
  auto kern = tc_gemm_kernel<LAYOUT, NMAT, NMAX>;
  using G = TcCfg<NMAX>;
  static bool configured[16] = {};
  int dev = 0;
  B200_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 16 && !configured[dev]) {
    B200_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM));
    configured[dev] = true;
  }
  kern<<<sm_count(), TC_THREADS, G::SMEM, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                                                maps[6], maps[7], maps[8], maps[9], a);
  B200_CHECK_CUDA(cudaGetLastError());
  return B200MOE_OK;
}

// The kernel variant follows the token tile: <= 64, <= 128 or <= 192 rows.
template <int LAYOUT, int NMAT>
int tc_launch(const CUtensorMap* maps, const TcArgs& a, cudaStream_t st) {
  if (a.tok_tile <= 64) return tc_launch_n<LAYOUT, NMAT, 64>(maps, a, st);
  if (a.tok_tile <= 128) return tc_launch_n<LAYOUT, NMAT, 128>(maps, a, st);
  return tc_launch_n<LAYOUT, NMAT, 192>(maps, a, st);
}

// Token tile for an expected number of rows per expert: experts with few rows
// stream their weights through the narrow, deeply buffered variants.  A
// segment longer than the tile simply takes several tiles.
int tc_pick_tok_tile(int tok_tile, int pairs, int experts) {
  const int est = pairs / (experts > 0 ? experts : 1);
  if (est <= 40) return tok_tile < 64 ? tok_tile : 64;
  if (est <= 96) return tok_tile < 128 ? tok_tile : 128;
  return tok_tile;
}

// Token-tile tensor maps with box heights 16, 32, 64, 96, 128 and 192 (maps[4..9]).
int tc_token_maps(CUtensorMap* maps, const void* x, int pairs, uint64_t row_bytes) {
  const int heights[6] = {16, 32, 64, 96, 128, 192};
  for (int i = 0; i < 6; ++i)
    if (int rc = make_tmap_2d_sw(&maps[4 + i], x, pairs, row_bytes, heights[i], 128, 128)) return rc;
  return B200MOE_OK;
}

int tc_check(const b200moe_weight_t* w, const char* name) {
  B200_REQUIRE(w->layout == B200MOE_LAYOUT_Q8_0 || w->layout == B200MOE_LAYOUT_Q4_K,
               "tensor kernel: %s must be Q8_0 or Q4_K (layout %d)", name, w->layout);
  B200_REQUIRE(w->cols % 256 == 0, "tensor kernel: %s cols (%d) must be a multiple of 256", name,
               w->cols);
  B200_REQUIRE(w->experts >= 1 && w->experts <= TC_MAX_E, "tensor kernel: %s experts out of range", name);
  const void* sc = w->layout == B200MOE_LAYOUT_Q8_0 ? w->d : w->sub;
  B200_REQUIRE(w->qs && sc && (reinterpret_cast<uintptr_t>(w->qs) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(sc) & 15) == 0,
               "tensor kernel: %s planes missing or misaligned", name);
  return B200MOE_OK;
}

int tc_weight_map(const b200moe_weight_t* w, CUtensorMap* tw, CUtensorMap* ts) {
  // 128-byte wide boxes of int8 with the 128-byte swizzle: 128 rows x 128 k;
  // scale boxes of 8 fp16 (256 k) x 128 rows, unswizzled
  const uint64_t rows = static_cast<uint64_t>(w->experts) * w->rows;
  if (w->layout == B200MOE_LAYOUT_Q4_K) {
    // nibbles: 64-byte wide boxes (128 k), 64-byte swizzle; (scale, min) pairs: 32 bytes per row
    if (int rc = make_tmap_2d_sw(tw, w->qs, rows, w->cols / 2, TC_ROWS, 64, 64)) return rc;
    return make_tmap_2d_sw(ts, w->sub, rows, static_cast<uint64_t>(w->cols) / 32 * 4, TC_ROWS, 32, 0);
  }
  if (int rc = make_tmap_2d_sw(tw, w->qs, rows, w->cols, TC_ROWS, 128, 128)) return rc;
  return make_tmap_2d_sw(ts, w->d, rows, static_cast<uint64_t>(w->cols) / 32 * 2, TC_ROWS, 16, 0);
}

}  // namespace

// Every shape condition the launchers below check, so that the automatic regime
// choice never picks the tensor kernel for a layer only the stream kernel can
// tile.  `down` selects the down projection's row rule (two 128-row sets of
// consecutive rows per tile) instead of the gate/up one (128 rows per set).
bool tc_supported(const b200moe_weight_t* w, bool down) {
  if (!(w->layout == B200MOE_LAYOUT_Q8_0 || w->layout == B200MOE_LAYOUT_Q4_K)) return false;
  if (w->cols % 256 != 0 || w->experts < 1 || w->experts > TC_MAX_E) return false;
  return w->rows % (down ? 2 * TC_ROWS : TC_ROWS) == 0;
}

int launch_tc_gate_up(const void* xs, const int32_t* seg, int pairs, int tok_tile,
                      const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                      int out_kperm, void* a_out, cudaStream_t st) {
  if (int rc = tc_check(gate, "gate")) return rc;
  if (int rc = tc_check(up, "up")) return rc;
  B200_REQUIRE(gate->rows == up->rows && gate->cols == up->cols && gate->experts == up->experts &&
                   gate->layout == up->layout,
               "tensor kernel: gate and up shapes or layouts differ");
  B200_REQUIRE(gate->rows % TC_ROWS == 0, "tensor kernel: ffn (%d) must be a multiple of 128", gate->rows);
  if (pairs == 0) return B200MOE_OK;
  CUtensorMap maps[10];
  if (int rc = tc_weight_map(gate, &maps[0], &maps[2])) return rc;
  if (int rc = tc_weight_map(up, &maps[1], &maps[3])) return rc;
  if (int rc = tc_token_maps(maps, xs, pairs, static_cast<uint64_t>(gate->cols) * 2)) return rc;
  TcArgs a{};
  a.seg = seg; a.E = gate->experts; a.N = gate->rows; a.K = gate->cols;
  a.ntiles = gate->rows / TC_ROWS; a.tok_tile = tc_pick_tok_tile(tok_tile, pairs, gate->experts); a.P = pairs; a.act = act;
  a.ksplit = 1;
  a.out_kperm = out_kperm;
  a.out = a_out; a.status = device_status_ptr();
  a.total_rows = static_cast<long long>(gate->experts) * gate->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  if (gate->layout == B200MOE_LAYOUT_Q4_K) return tc_launch<B200MOE_LAYOUT_Q4_K, 2>(maps, a, st);
  if (gate->sub != nullptr && up->sub != nullptr) {
    a.st0 = static_cast<const uint8_t*>(gate->sub);
    a.st1 = static_cast<const uint8_t*>(up->sub);
  }
  return tc_launch<B200MOE_LAYOUT_Q8_0, 2>(maps, a, st);
}

int tc_down_ksplit(const b200moe_weight_t* down, int est_pairs) {
  // Few tiles (expert-parallel ranks with one or two experts) leave SMs idle:
  // split the long reduction into up to four partitions when that fills the
  // waves better.  est_pairs is the expected number of rows, not a bound.
  const int stages = down->cols / TC_KT;
  const int sms = sm_count();
  const int per_expert = est_pairs / (down->experts > 0 ? down->experts : 1);
  const long long tiles = static_cast<long long>(down->experts) * (down->rows / (2 * TC_ROWS)) *
                          ((per_expert + 191) / 192 > 0 ? (per_expert + 191) / 192 : 1);
  if (tiles >= 2ll * sms) return 1;
  int best = 1;
  double best_eff = 0.0;
  for (int ks = 1; ks <= 4; ks *= 2) {
    if (stages % (4 * ks) != 0) break;
    const long long items = tiles * ks;
    const long long waves = (items + sms - 1) / sms;
    const double eff = static_cast<double>(items) / (waves * sms) - 0.03 * (ks - 1);
    if (eff > best_eff) { best_eff = eff; best = ks; }
  }
  return best;
}

int launch_tc_down(const void* a_in, const int32_t* seg, int pairs, int tok_tile,
                   const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st) {
  if (int rc = tc_check(down, "down")) return rc;
  B200_REQUIRE(down->rows % (2 * TC_ROWS) == 0, "tensor kernel: hidden (%d) must be a multiple of 256",
               down->rows);
  if (pairs == 0) return B200MOE_OK;
  CUtensorMap maps[10];
  if (int rc = tc_weight_map(down, &maps[0], &maps[2])) return rc;
  maps[1] = maps[0];
  maps[3] = maps[2];
  if (int rc = tc_token_maps(maps, a_in, pairs, static_cast<uint64_t>(down->cols) * 2)) return rc;
  TcArgs a{};
  a.seg = seg; a.E = down->experts; a.N = down->rows; a.K = down->cols;
  B200_REQUIRE(ksplit >= 1 && (down->cols / TC_KT) % (4 * ksplit) == 0, "tensor kernel: bad k split %d",
               ksplit);
  a.ntiles = down->rows / (2 * TC_ROWS); a.tok_tile = tc_pick_tok_tile(tok_tile, pairs, down->experts); a.P = pairs; a.act = 0;
  a.ksplit = ksplit;
  a.out = d_out; a.status = device_status_ptr();
  a.total_rows = static_cast<long long>(down->experts) * down->rows;
  if (a.status == nullptr) return B200MOE_ERR_CUDA;
  if (down->layout == B200MOE_LAYOUT_Q4_K) return tc_launch<B200MOE_LAYOUT_Q4_K, 1>(maps, a, st);
  if (down->sub != nullptr) a.st0 = a.st1 = static_cast<const uint8_t*>(down->sub);
  return tc_launch<B200MOE_LAYOUT_Q8_0, 1>(maps, a, st);
}

}  // namespace b200moe
