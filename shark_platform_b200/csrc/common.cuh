// Shared host/device helpers: error reporting, PTX wrappers for mbarrier / TMA /
// mma.sync, and the tensor-map encoder fetched from the driver at run time.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
// Device status word of the current device (kernels OR their error codes in).
int32_t* device_status_ptr();
int sm_count();

#define B200_CHECK_CUDA(expr)                                   \
  do {                                                          \
    cudaError_t _e = (expr);                                    \
    if (_e != cudaSuccess) return ::b200moe::cuda_fail(_e, #expr); \
  } while (0)

#define B200_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      ::b200moe::set_error(__VA_ARGS__);   \
      return B200MOE_ERR_INVALID;          \
    }                                      \
  } while (0)

// 2-D tiled tensor map over a row-major [rows, cols] array of `elem_bytes`
// elements.  box = {box_cols, box_rows}; swizzle128 selects the 128-byte
// shared-memory swizzle (box_cols*elem_bytes must then be 128).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                 uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                 bool swizzle128);

// Same over a byte array: row_bytes per row, a box of box_rows x box_bytes and
// a shared-memory swizzle of 0, 32, 64 or 128 bytes (box_bytes <= swizzle).
int make_tmap_2d_sw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes,
                    uint32_t box_rows, uint32_t box_bytes, int swizzle_bytes);

// Error bits written to the device status word.
enum : int32_t {
  DEV_ERR_WAIT_TIMEOUT = 1,  // a bounded mbarrier wait gave up
  DEV_ERR_BOUNDS = 2,        // an index check failed; the access was skipped
  DEV_ERR_TMEM = 4,          // tensor-memory allocation/wait gave up
  DEV_ERR_MASK = 7,
  DEV_WARN_SATURATED = 8,    // an fp16 operand was clipped to +-65504 (a warning, not an error)
};

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders this thread's generic-proxy shared-memory accesses (ld.shared /
// st.shared) against async-proxy accesses (TMA).  A buffer that TMA refills
// needs it on the release path as well: ld.shared reads followed by a TMA
// write of the same bytes are a cross-proxy write-after-read, which the
// mbarrier release/acquire pair alone does not order.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Gives up after ~2^31 clock ticks (about a second), records
// DEV_ERR_WAIT_TIMEOUT in the status word and raises the CTA-wide abort flag so
// that every later wait in this CTA returns at once.  Returns false on abort.
// The barrier is tried first: a phase that has already completed costs one
// try_wait and no shared-memory load of the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > (1ll << 31)) {
      *abort_flag = 1;
      atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
      return false;
    }
  }
}

// The same wait for a whole warp (all 32 lanes call it, converged).  Every lane
// runs its own bounded wait, so all of them come back; the vote then makes the
// outcome uniform: when the abort flag is raised at the moment a phase completes,
// one lane may see the phase and another the flag, and a warp that split on that
// would meet `.sync.aligned` instructions or block-wide barriers with lanes
// missing.  Either every lane continues or every lane gives up.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int* abort_flag, int32_t* status) {
  const bool ok = mbar_wait(bar, parity, abort_flag, status);
  return __all_sync(0xffffffffu, ok);
}

// 2-D tiled bulk tensor load global -> shared, completion on an mbarrier.
// x = innermost (column) coordinate in elements; x*elem_bytes must be a
// multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, int32_t x,
                                            int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t (&v)[4]) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void lds64(uint32_t addr, uint32_t (&v)[2]) {
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint32_t (&v)[4]) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v[0]), "r"(v[1]),
               "r"(v[2]), "r"(v[3])
               : "memory");
}

// D += A(16x16, row) * B(16x8, col), fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}

// Four int8 (one 32-bit word, k order = byte order) -> four fp16 values times
// the block scale, as two half2: lo = (k0,k1), hi = (k2,k3).  Each product is
// fp16(d*q): 0x6400|b is the fp16 number 1024+b, so after biasing the byte to
// unsigned the subtraction of 1152 yields q exactly, and one rounded multiply
// follows — the same value as `d.to(fp16) * qs.to(fp16)`.
__device__ __forceinline__ void dequant_q8x4(uint32_t w, __half2 scale, uint32_t& lo,
                                             uint32_t& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const __half2 bias = u32_as_h2(0x64806480u);  // 1152, 1152
  const __half2 l = __hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4140)), bias);
  const __half2 h = __hsub2(u32_as_h2(__byte_perm(x, 0x64646464u, 0x4342)), bias);
  lo = h2_as_u32(__hmul2(l, scale));
  hi = h2_as_u32(__hmul2(h, scale));
}

// Eight 4-bit quants of one 32-bit word (k order: nibble i of byte b is
// element 2b+i) -> fp16(fp16(ds*q) - dm) as four half2 whose element pairs are
// (q0,q4) (q1,q5) (q2,q6) (q3,q7): the pair order the activation rows are
// pre-permuted to.  0x6400|q is the fp16 number 1024+q, and -1024*ds is exact in
// fp16 (a power-of-two multiple; ds < 64), so one fused multiply-add
// (1024+q)*ds - 1024*ds is the exact product ds*q rounded once — the value of the
// reference's fp16 multiply — without first subtracting the 1024.  The offset is
// then subtracted with its own rounding (_rn: never contracted into the fma).
__device__ __forceinline__ void dequant_q4x8(uint32_t w, __half2 ds, __half2 dm,
                                             uint32_t (&out)[4]) {
  const __half2 nds1024 = __hmul2(ds, u32_as_h2(0xE400E400u));  // -1024 * ds, exact
  const uint32_t w1 = w >> 8;
  uint32_t e[4];
  e[0] = (w & 0x000f000fu) | 0x64006400u;          // (q0, q4)
  e[1] = ((w >> 4) & 0x000f000fu) | 0x64006400u;   // (q1, q5)
  e[2] = (w1 & 0x000f000fu) | 0x64006400u;         // (q2, q6)
  e[3] = ((w1 >> 4) & 0x000f000fu) | 0x64006400u;  // (q3, q7)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 t = __hfma2(u32_as_h2(e[i]), ds, nds1024);
    out[i] = h2_as_u32(__hsub2_rn(t, dm));
  }
}

// x * sigmoid(x) with the approximate exponential and reciprocal (two special-
// function instructions, relative error ~1e-6: far below the fp16 rounding of
// the product that follows); an IEEE division costs several times as much and
// the epilogue of a 128 x 192 tile evaluates 24576 of these.
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float gelu_erf_f(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

// fp32 -> fp16 with saturation to the largest finite value (no infinities in
// the expert operand).
__device__ __forceinline__ __half to_half_sat(float v) {
  v = fminf(fmaxf(v, -65504.0f), 65504.0f);
  return __float2half_rn(v);
}

// The same, recording in the status word that a value was out of fp16 range
// (|v| >= 65520 would round to infinity; NaN is passed through unflagged).
__device__ __forceinline__ __half to_half_sat(float v, int32_t* status) {
  if (fabsf(v) >= 65520.0f) atomicOr(status, DEV_WARN_SATURATED);
  return to_half_sat(v);
}

#endif  // __CUDACC__

}  // namespace b200moe
