// C ABI of the library: argument checking, workspace carving and the sequence
// of kernel launches that makes up one MoE layer call.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "kernels.h"

namespace b200moe {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return B200MOE_ERR_CUDA;
}

// Device status word: one per device, lives in the module's global memory.
__device__ int32_t g_device_status = 0;

int32_t* device_status_ptr() {
  static int32_t* ptrs[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
    set_error("device_status_ptr: no usable current device");
    return nullptr;
  }
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_device_status);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaGetSymbolAddress(g_device_status)");
      return nullptr;
    }
    ptrs[dev] = static_cast<int32_t*>(p);
  }
  return ptrs[dev];
}

int sm_count() {
  static int counts[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 148;
  if (counts[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    counts[dev] = n;
  }
  return counts[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_2d_sw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes,
                    uint32_t box_rows, uint32_t box_bytes, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return B200MOE_ERR_CUDA;
  }
  B200_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor map base misaligned");
  B200_REQUIRE(row_bytes % 16 == 0, "tensor map row pitch must be a multiple of 16 bytes");
  B200_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_bytes >= 16 && box_bytes <= 256 &&
                   box_bytes % 16 == 0,
               "tensor map box out of range");
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  else if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  else if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  else B200_REQUIRE(swizzle_bytes == 0, "tensor map swizzle must be 0, 32, 64 or 128");
  B200_REQUIRE(swizzle_bytes == 0 || box_bytes <= static_cast<uint32_t>(swizzle_bytes),
               "tensor map box row wider than the swizzle span");
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d (rows=%llu row_bytes=%llu box=%ux%u)",
              static_cast<int>(r), static_cast<unsigned long long>(rows),
              static_cast<unsigned long long>(row_bytes), box_rows, box_bytes);
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                 uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                 bool swizzle128) {
  (void)dt;
  B200_REQUIRE(!swizzle128 || box_cols * elem_bytes == 128, "128B swizzle needs a 128-byte box row");
  return make_tmap_2d_sw(out, base, rows, cols * elem_bytes, box_rows, box_cols * elem_bytes,
                         swizzle128 ? 128 : 0);
}

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Upper bound of the tensor kernels' token tile (b200moe_set_token_tile).
int g_token_tile = 192;

// Above this many tokens the tensor-memory kernel takes over from the
// weight-streaming kernel (where the layout allows it).
constexpr int TENSOR_MIN_TOKENS = 97;

// `down` says which of the two products the weight belongs to (their tile
// shapes differ).  An explicit regime is taken as given and fails in the
// launcher when the shape does not fit; AUTO only picks what can run.
int pick_regime(int regime, const b200moe_weight_t* w, int max_segment, bool down) {
  if (regime == B200MOE_REGIME_TENSOR) return B200MOE_REGIME_TENSOR;
  if (regime == B200MOE_REGIME_TENSOR_PAIR) return B200MOE_REGIME_TENSOR_PAIR;
  if (regime == B200MOE_REGIME_STREAM) return B200MOE_REGIME_STREAM;
  const bool can_tensor = w != nullptr && tc_supported(w, down);
  return (can_tensor && max_segment >= TENSOR_MIN_TOKENS) ? B200MOE_REGIME_TENSOR
                                                          : B200MOE_REGIME_STREAM;
}

// Workspace carve-up of one layer call.
struct Workspace {
  __half* xn;
  int32_t* experts;
  float* gates;
  int32_t* counts;
  int32_t* seg;
  int32_t* perm;
  int32_t* inv;
  __half* xs;
  __half* a;
  float* dpart;
  size_t bytes;
};

Workspace carve(const b200moe_layer_t* L, int tokens, void* base) {
  const size_t T = tokens > 0 ? tokens : 1;
  const size_t P = T * L->top_k;
  const size_t d = L->hidden, F = L->ffn;
  int ks = stream_down_ksplit(&L->down, static_cast<int>(P));
  if (tc_supported(&L->down, true)) ks = max(ks, tc_down_ksplit(&L->down, static_cast<int>(P)));
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t n) {
    void* r = p ? p + off : nullptr;
    off += align_up(n, 1024);
    return r;
  };
  Workspace w;
  w.xn = static_cast<__half*>(take(T * d * 2));
  w.experts = static_cast<int32_t*>(take(P * 4));
  w.gates = static_cast<float*>(take(P * 4));
  w.counts = static_cast<int32_t*>(take(64 * 4));
  w.seg = static_cast<int32_t*>(take(65 * 4));
  w.perm = static_cast<int32_t*>(take(P * 4));
  w.inv = static_cast<int32_t*>(take(P * 4));
  w.xs = static_cast<__half*>(take(P * d * 2));
  w.a = static_cast<__half*>(take(P * F * 2));
  w.dpart = static_cast<float*>(take(static_cast<size_t>(ks) * P * d * 4));
  w.bytes = off;
  return w;
}

int check_layer(const b200moe_layer_t* L) {
  B200_REQUIRE(L != nullptr, "layer is NULL");
  B200_REQUIRE(L->hidden > 0 && L->ffn > 0, "layer: bad sizes");
  B200_REQUIRE(L->gate.rows == L->ffn && L->gate.cols == L->hidden, "layer: gate shape mismatch");
  B200_REQUIRE(L->up.rows == L->ffn && L->up.cols == L->hidden, "layer: up shape mismatch");
  B200_REQUIRE(L->down.rows == L->hidden && L->down.cols == L->ffn, "layer: down shape mismatch");
  B200_REQUIRE(L->gate.experts == L->up.experts && L->gate.experts == L->down.experts,
               "layer: expert counts differ between matrices");
  B200_REQUIRE(L->expert_begin >= 0 && L->expert_begin + L->gate.experts <= L->experts,
               "layer: local expert range outside [0, experts)");
  B200_REQUIRE(L->ffn_norm_weight && L->router_weight, "layer: missing norm or router weight");
  return B200MOE_OK;
}

// Stage profiler: a ring of event sets, one set of 7 events per recorded call.
constexpr int PROF_STAGES = 6;
constexpr int PROF_CALLS = 512;
struct Profiler {
  bool on = false;
  int used = 0;
  cudaEvent_t ev[PROF_CALLS][PROF_STAGES + 1] = {};
  bool created = false;
};
Profiler g_prof;

inline void prof_mark(int call, int idx, cudaStream_t st) {
  if (call >= 0) cudaEventRecord(g_prof.ev[call][idx], st);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

const char* b200moe_version(void) { return "b200moe 0.1 (sm_100a)"; }
const char* b200moe_last_error(void) { return g_error; }

int b200moe_device_status(void* stream, int32_t* status_out) {
  int32_t* p = device_status_ptr();
  if (p == nullptr) return B200MOE_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t v = 0;
  B200_CHECK_CUDA(cudaMemcpyAsync(&v, p, sizeof(v), cudaMemcpyDeviceToHost, st));
  B200_CHECK_CUDA(cudaMemsetAsync(p, 0, sizeof(v), st));
  B200_CHECK_CUDA(cudaStreamSynchronize(st));
  if (status_out) *status_out = v;
  if ((v & DEV_ERR_MASK) != 0) {
    clear_front_sync(st);  // a timed-out grid barrier leaves its counters behind
    cudaStreamSynchronize(st);
    set_error("device status word = %d (1: bounded wait timed out, 2: bounds check, 4: tmem, "
              "8: fp16 operand clipped)", v);
    return B200MOE_ERR_DEVICE;
  }
  return B200MOE_OK;
}

int b200moe_front_supported(int32_t tokens, const b200moe_layer_t* layer) {
  return layer != nullptr && front_fused_supported(tokens, layer) ? 1 : 0;
}

int b200moe_front(const void* h, int h_dtype, int32_t tokens, const b200moe_layer_t* layer,
                  int kperm, int32_t* experts_out, float* gates_out, int32_t* counts,
                  int32_t* seg_offsets, int32_t* perm, int32_t* inv, void* xs_out, void* stream) {
  B200_REQUIRE(layer, "front: NULL layer");
  B200_REQUIRE(layer->ffn_norm_weight && layer->router_weight, "front: NULL router parameters");
  B200_REQUIRE(h && experts_out && gates_out && counts && seg_offsets && perm && inv && xs_out,
               "front: NULL buffer");
  int32_t* status = device_status_ptr();
  if (status == nullptr) return B200MOE_ERR_CUDA;
  return launch_front_fused(h, h_dtype, tokens, layer, experts_out, gates_out, counts, seg_offsets,
                            perm, inv, kperm != 0, xs_out, status, static_cast<cudaStream_t>(stream));
}

int b200moe_dequant(const b200moe_weight_t* w, int out_dtype, void* out, void* stream) {
  B200_REQUIRE(w && out, "dequant: NULL argument");
  return launch_dequant(w, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200moe_q4k_prepare(const void* d, const void* dmin, const uint8_t* sh, const uint8_t* sl,
                        const uint8_t* mh, const uint8_t* ml, int64_t blocks, void* sub_out,
                        void* stream) {
  B200_REQUIRE(blocks >= 0, "q4k_prepare: negative block count");
  B200_REQUIRE(blocks == 0 || (d && dmin && sh && sl && mh && ml && sub_out),
               "q4k_prepare: NULL argument");
  return launch_q4k_prepare(d, dmin, sh, sl, mh, ml, blocks, sub_out,
                            static_cast<cudaStream_t>(stream));
}

int b200moe_q8_prepare(const void* d, int64_t rows, int32_t cols, void* sub_out, void* stream) {
  B200_REQUIRE(rows >= 0 && (rows == 0 || (d && sub_out)), "q8_prepare: bad argument");
  return launch_q8_prepare(d, rows, cols, sub_out, static_cast<cudaStream_t>(stream));
}

int b200moe_gguf_unpack_q8_0(const uint8_t* raw, int64_t blocks, void* d_out, int8_t* qs_out,
                             void* stream) {
  B200_REQUIRE(blocks >= 0 && (blocks == 0 || (raw && d_out && qs_out)), "gguf_unpack_q8_0: bad argument");
  return launch_gguf_q8(raw, blocks, d_out, qs_out, static_cast<cudaStream_t>(stream));
}

int b200moe_gguf_unpack_q4_k(const uint8_t* raw, int64_t blocks, void* d_out, void* dmin_out,
                             uint8_t* sh, uint8_t* sl, uint8_t* mh, uint8_t* ml, uint8_t* qs_out,
                             void* stream) {
  B200_REQUIRE(blocks >= 0 && (blocks == 0 || (raw && d_out && dmin_out && sh && sl && mh && ml && qs_out)),
               "gguf_unpack_q4_k: bad argument");
  return launch_gguf_q4k(raw, blocks, d_out, dmin_out, sh, sl, mh, ml, qs_out,
                         static_cast<cudaStream_t>(stream));
}

int b200moe_router(const void* h, int h_dtype, int32_t tokens, const b200moe_layer_t* layer,
                   void* xn_out, int32_t* experts_out, float* gates_out, void* stream) {
  B200_REQUIRE(layer && tokens >= 0, "router: bad argument");
  B200_REQUIRE(tokens == 0 || (h && xn_out && experts_out && gates_out), "router: NULL buffer");
  return launch_router(h, h_dtype, tokens, layer, xn_out, experts_out, gates_out,
                       static_cast<cudaStream_t>(stream));
}

int b200moe_route_plan(const int32_t* experts, int32_t pairs, int32_t expert_begin,
                       int32_t experts_local, int32_t* counts, int32_t* seg_offsets,
                       int32_t* perm, int32_t* inv, void* stream) {
  B200_REQUIRE(counts && seg_offsets, "route_plan: NULL output");
  B200_REQUIRE(pairs == 0 || (experts && perm && inv), "route_plan: NULL buffer");
  return launch_route_plan(experts, pairs, expert_begin, experts_local, counts, seg_offsets, perm,
                           inv, static_cast<cudaStream_t>(stream));
}

int b200moe_permute_rows(const void* xn, const int32_t* perm, const int32_t* seg_offsets,
                         int32_t experts_local, int32_t pairs, int32_t top_k, int32_t hidden,
                         int32_t kperm, void* xs_out, void* stream) {
  B200_REQUIRE(pairs == 0 || (xn && perm && seg_offsets && xs_out), "permute_rows: NULL buffer");
  B200_REQUIRE(top_k >= 1, "permute_rows: top_k must be positive");
  return launch_permute_rows(xn, perm, seg_offsets, experts_local, pairs, top_k, hidden, kperm,
                             xs_out, static_cast<cudaStream_t>(stream));
}

int b200moe_kperm(int layout, int regime, int32_t max_segment) {
  (void)regime;
  (void)max_segment;
  // both Q4_K kernels pull nibble pairs (q_i, q_i+4) out of a word and want
  // the matching column interleave
  return layout == B200MOE_LAYOUT_Q4_K ? 1 : 0;
}

int b200moe_gate_up(const void* xs, const int32_t* seg_offsets, int32_t pairs,
                    int32_t max_segment, const b200moe_weight_t* gate,
                    const b200moe_weight_t* up, int activation, int regime, int32_t out_kperm,
                    void* a_out, void* stream) {
  B200_REQUIRE(gate && up && seg_offsets, "gate_up: NULL argument");
  B200_REQUIRE(pairs == 0 || (xs && a_out), "gate_up: NULL buffer");
  B200_REQUIRE(activation == B200MOE_ACT_SILU || activation == B200MOE_ACT_GELU,
               "gate_up: unknown activation %d", activation);
  int r = pick_regime(regime, gate, max_segment, false);
  // shapes the pair kernel cannot tile go to the single-CTA tensor kernel
  if (r == B200MOE_REGIME_TENSOR_PAIR && !(tc_pair_supported_gate_up(gate) && tc_pair_supported_gate_up(up)))
    r = B200MOE_REGIME_TENSOR;
  if (r == B200MOE_REGIME_TENSOR_PAIR)
    return launch_tc_pair_gate_up(xs, seg_offsets, pairs, 192, gate, up, activation, out_kperm, a_out,
                                  static_cast<cudaStream_t>(stream));
  if (r == B200MOE_REGIME_TENSOR) {
    return launch_tc_gate_up(xs, seg_offsets, pairs, g_token_tile, gate, up, activation, out_kperm, a_out,
                             static_cast<cudaStream_t>(stream));
  }
  return launch_stream_gate_up(xs, seg_offsets, pairs, max_segment, gate, up, activation,
                               out_kperm, a_out, static_cast<cudaStream_t>(stream));
}

int b200moe_down_ksplit(const b200moe_weight_t* down, int32_t pairs, int32_t max_segment,
                        int regime) {
  if (down == nullptr) return 1;
  int r = pick_regime(regime, down, max_segment, true);
  if (r == B200MOE_REGIME_TENSOR_PAIR && !tc_pair_supported_down(down)) r = B200MOE_REGIME_TENSOR;
  if (r == B200MOE_REGIME_TENSOR_PAIR) return 1;
  if (r == B200MOE_REGIME_TENSOR) return tc_down_ksplit(down, pairs);
  return stream_down_ksplit(down, pairs);
}

int b200moe_down(const void* a, const int32_t* seg_offsets, int32_t pairs, int32_t max_segment,
                 const b200moe_weight_t* down, int regime, int32_t ksplit, float* d_out,
                 void* stream) {
  B200_REQUIRE(down && seg_offsets, "down: NULL argument");
  B200_REQUIRE(pairs == 0 || (a && d_out), "down: NULL buffer");
  B200_REQUIRE(ksplit >= 1, "down: ksplit must come from b200moe_down_ksplit");
  int r = pick_regime(regime, down, max_segment, true);
  if (r == B200MOE_REGIME_TENSOR_PAIR && !tc_pair_supported_down(down)) r = B200MOE_REGIME_TENSOR;
  if (r == B200MOE_REGIME_TENSOR_PAIR)
    return launch_tc_pair_down(a, seg_offsets, pairs, 192, down, ksplit, d_out,
                               static_cast<cudaStream_t>(stream));
  if (r == B200MOE_REGIME_TENSOR)
    return launch_tc_down(a, seg_offsets, pairs, g_token_tile, down, ksplit, d_out,
                          static_cast<cudaStream_t>(stream));
  return launch_stream_down(a, seg_offsets, pairs, max_segment, down, ksplit, d_out,
                            static_cast<cudaStream_t>(stream));
}

int b200moe_exchange_plan(const int32_t* counts, int32_t world, int32_t experts_local,
                          int32_t* seg_offsets, int32_t* perm, int32_t* inv, void* stream) {
  B200_REQUIRE(counts && seg_offsets && perm && inv, "exchange_plan: NULL argument");
  return launch_exchange_plan(counts, world, experts_local, seg_offsets, perm, inv,
                              static_cast<cudaStream_t>(stream));
}

int b200moe_gather_rows(const void* rows, const int32_t* idx, int32_t n, int32_t div,
                        int32_t row_bytes, void* out, void* stream) {
  B200_REQUIRE(n >= 0 && (n == 0 || (rows && idx && out)), "gather_rows: bad argument");
  return launch_gather_rows(rows, idx, n, div, row_bytes, out, static_cast<cudaStream_t>(stream));
}

int b200moe_combine(const void* d_partials, int d_dtype, int32_t ksplit, int32_t pairs, const int32_t* inv,
                    const float* gates, const void* h, int h_dtype, int32_t tokens,
                    const b200moe_layer_t* layer, int add_residual, void* y_out, int y_dtype,
                    void* stream) {
  B200_REQUIRE(layer && ksplit >= 1, "combine: bad argument");
  B200_REQUIRE(tokens == 0 || (d_partials && inv && gates && y_out), "combine: NULL buffer");
  B200_REQUIRE(!add_residual || h, "combine: residual requested without h");
  return launch_combine(d_partials, d_dtype, ksplit, pairs, inv, gates, h, h_dtype, tokens, layer,
                        add_residual, y_out, y_dtype, static_cast<cudaStream_t>(stream));
}

size_t b200moe_workspace_bytes(const b200moe_layer_t* layer, int32_t tokens) {
  if (layer == nullptr || tokens < 0) return 0;
  return carve(layer, tokens, nullptr).bytes;
}

int b200moe_layer_forward(const b200moe_layer_t* L, const void* h, void* y, int io_dtype,
                          int32_t tokens, int regime, void* workspace, size_t workspace_bytes,
                          int32_t* experts_out, float* gates_out, void* stream) {
  if (int rc = check_layer(L)) return rc;
  B200_REQUIRE(tokens >= 0, "layer_forward: negative token count");
  if (tokens == 0) return B200MOE_OK;
  B200_REQUIRE(h && y && workspace, "layer_forward: NULL buffer");
  B200_REQUIRE(io_dtype == B200MOE_DT_F32 || io_dtype == B200MOE_DT_BF16,
               "layer_forward: activations must be fp32 or bf16");
  B200_REQUIRE(L->gate.experts == L->experts && L->expert_begin == 0,
               "layer_forward: expert-sharded layers go through the staged entry points");
  Workspace w = carve(L, tokens, workspace);
  if (w.bytes > workspace_bytes) {
    set_error("layer_forward: workspace needs %zu bytes, got %zu", w.bytes, workspace_bytes);
    return B200MOE_ERR_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int pairs = tokens * L->top_k;
  const int E = L->experts;
  const int pc = (g_prof.on && g_prof.used < PROF_CALLS) ? g_prof.used++ : -1;
  const int kp_in = b200moe_kperm(L->gate.layout, regime, tokens);
  const int kp_mid = b200moe_kperm(L->down.layout, regime, tokens);
  prof_mark(pc, 0, st);
  if (front_fused_supported(tokens, L)) {
    // decode: one launch; its time is booked under the router stage
    int32_t* status = device_status_ptr();
    if (status == nullptr) return B200MOE_ERR_CUDA;
    if (int rc = launch_front_fused(h, io_dtype, tokens, L, w.experts, w.gates, w.counts, w.seg,
                                    w.perm, w.inv, kp_in, w.xs, status, st))
      return rc;
    prof_mark(pc, 1, st);
    prof_mark(pc, 2, st);
  } else {
    if (int rc = launch_router(h, io_dtype, tokens, L, w.xn, w.experts, w.gates, st)) return rc;
    prof_mark(pc, 1, st);
    if (int rc = launch_route_plan(w.experts, pairs, 0, E, w.counts, w.seg, w.perm, w.inv, st))
      return rc;
    prof_mark(pc, 2, st);
    if (int rc = launch_permute_rows(w.xn, w.perm, w.seg, E, pairs, L->top_k, L->hidden, kp_in, w.xs, st))
      return rc;
  }
  prof_mark(pc, 3, st);
  if (int rc = b200moe_gate_up(w.xs, w.seg, pairs, tokens, &L->gate, &L->up, L->activation, regime,
                               kp_mid, w.a, stream))
    return rc;
  prof_mark(pc, 4, st);
  const int ks = b200moe_down_ksplit(&L->down, pairs, tokens, regime);
  if (int rc = b200moe_down(w.a, w.seg, pairs, tokens, &L->down, regime, ks, w.dpart, stream)) return rc;
  prof_mark(pc, 5, st);
  if (int rc = launch_combine(w.dpart, B200MOE_DT_F32, ks, pairs, w.inv, w.gates, h, io_dtype,
                              tokens, L, 1, y, io_dtype, st))
    return rc;
  prof_mark(pc, 6, st);
  if (experts_out)
    B200_CHECK_CUDA(cudaMemcpyAsync(experts_out, w.experts, sizeof(int32_t) * pairs,
                                    cudaMemcpyDeviceToDevice, st));
  if (gates_out)
    B200_CHECK_CUDA(cudaMemcpyAsync(gates_out, w.gates, sizeof(float) * pairs,
                                    cudaMemcpyDeviceToDevice, st));
  return B200MOE_OK;
}

int b200moe_layer_forward_host(const b200moe_layer_t* L, const void* h_host, void* y_host,
                               int io_dtype, int32_t tokens, int regime, void* dev_io,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_layer(L)) return rc;
  B200_REQUIRE(tokens >= 0, "layer_forward_host: negative token count");
  if (tokens == 0) return B200MOE_OK;
  B200_REQUIRE(h_host && y_host && dev_io, "layer_forward_host: NULL buffer");
  B200_REQUIRE(io_dtype == B200MOE_DT_F32 || io_dtype == B200MOE_DT_BF16,
               "layer_forward_host: activations must be fp32 or bf16");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(tokens) * L->hidden * (io_dtype == B200MOE_DT_F32 ? 4 : 2);
  uint8_t* dh = static_cast<uint8_t*>(dev_io);
  uint8_t* dy = dh + align_up(bytes, 1024);
  B200_CHECK_CUDA(cudaMemcpyAsync(dh, h_host, bytes, cudaMemcpyHostToDevice, st));
  if (int rc = b200moe_layer_forward(L, dh, dy, io_dtype, tokens, regime, workspace,
                                     workspace_bytes, nullptr, nullptr, stream))
    return rc;
  B200_CHECK_CUDA(cudaMemcpyAsync(y_host, dy, bytes, cudaMemcpyDeviceToHost, st));
  return B200MOE_OK;
}

// ---- expert parallelism: the whole per-layer sequence from one call ---------
namespace {
struct EpWorkspace {
  __half* xn;
  int32_t* experts;
  float* gates;
  int32_t* counts;
  int32_t* seg;
  int32_t* perm;
  int32_t* inv;
  int32_t* seg2;
  __half* a;
  float* dpart;
  size_t bytes;
};

EpWorkspace ep_carve(const b200moe_layer_t* L, int tokens, int cap_rows, int ksplit, void* base) {
  const size_t T = tokens > 0 ? tokens : 1;
  const size_t P = T * L->top_k;
  const size_t R = cap_rows > 0 ? cap_rows : 1;
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t n) {
    void* r = p ? p + off : nullptr;
    off += align_up(n, 1024);
    return r;
  };
  EpWorkspace w;
  w.xn = static_cast<__half*>(take(T * L->hidden * 2));
  w.experts = static_cast<int32_t*>(take(P * 4));
  w.gates = static_cast<float*>(take(P * 4));
  w.counts = static_cast<int32_t*>(take(64 * 4));
  w.seg = static_cast<int32_t*>(take(65 * 4));
  w.perm = static_cast<int32_t*>(take(P * 4));
  w.inv = static_cast<int32_t*>(take(P * 4));
  w.seg2 = static_cast<int32_t*>(take(65 * 4));
  w.a = static_cast<__half*>(take(R * L->ffn * 2));
  w.dpart = static_cast<float*>(take(static_cast<size_t>(ksplit) * R * L->hidden * 4));
  w.bytes = off;
  return w;
}
}  // namespace

size_t b200moe_ep_workspace_bytes(const b200moe_layer_t* layer, int32_t tokens, int32_t cap_rows,
                                  int32_t ksplit) {
  if (layer == nullptr || tokens < 0 || cap_rows < 0 || ksplit < 1) return 0;
  return ep_carve(layer, tokens, cap_rows, ksplit, nullptr).bytes;
}

int b200moe_ep_layer_forward(const b200moe_layer_t* L, const b200moe_ep_t* ep, const void* h, void* y,
                             int io_dtype, int32_t tokens, int regime, int32_t cap_rows,
                             int32_t ret_rows, int32_t max_segment, int32_t ksplit, int32_t epoch,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_layer(L)) return rc;
  B200_REQUIRE(ep != nullptr, "ep_layer_forward: NULL exchange descriptor");
  B200_REQUIRE(ep->world >= 1 && ep->rank >= 0 && ep->rank < ep->world && ep->world <= 16,
               "ep_layer_forward: world %d / rank %d out of range", ep->world, ep->rank);
  B200_REQUIRE(L->gate.experts == ep->experts_local && L->experts == ep->experts_local * ep->world &&
                   L->expert_begin == ep->rank * ep->experts_local,
               "ep_layer_forward: the layer must hold this rank's expert shard "
               "(experts_local %d, begin %d of %d)", L->gate.experts, L->expert_begin, L->experts);
  B200_REQUIRE(tokens >= 0 && cap_rows >= 1 && ksplit >= 1 && max_segment >= 1,
               "ep_layer_forward: bad sizes");
  B200_REQUIRE(tokens * L->top_k <= ret_rows, "ep_layer_forward: %d pairs exceed the return buffer (%d rows)",
               tokens * L->top_k, ret_rows);
  B200_REQUIRE(io_dtype == B200MOE_DT_F32 || io_dtype == B200MOE_DT_BF16,
               "ep_layer_forward: activations must be fp32 or bf16");
  B200_REQUIRE((tokens == 0 || (h && y)) && workspace, "ep_layer_forward: NULL buffer");
  EpWorkspace w = ep_carve(L, tokens, cap_rows, ksplit, workspace);
  if (w.bytes > workspace_bytes) {
    set_error("ep_layer_forward: workspace needs %zu bytes, got %zu", w.bytes, workspace_bytes);
    return B200MOE_ERR_WORKSPACE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int pairs = tokens * L->top_k;
  const int E = L->experts;
  const int pc = (g_prof.on && g_prof.used < PROF_CALLS) ? g_prof.used++ : -1;
  const int kp_in = b200moe_kperm(L->gate.layout, regime, max_segment);
  const int kp_mid = b200moe_kperm(L->down.layout, regime, max_segment);
  void* recv_x = ep->recv_x[ep->rank];
  void* ret_y = ep->ret_y[ep->rank];
  // every rank takes part in every barrier, also one that has no tokens
  prof_mark(pc, 0, st);
  if (tokens > 0)
    if (int rc = launch_router(h, io_dtype, tokens, L, w.xn, w.experts, w.gates, st)) return rc;
  prof_mark(pc, 1, st);
  if (int rc = launch_route_plan(w.experts, pairs, 0, E, w.counts, w.seg, w.perm, w.inv, st)) return rc;
  if (int rc = b200moe_ep_publish_counts(ep, w.counts, stream)) return rc;
  if (int rc = b200moe_ep_barrier(ep, epoch + 1, w.seg2, stream)) return rc;
  prof_mark(pc, 2, st);
  if (int rc = b200moe_ep_dispatch(ep, w.xn, w.experts, w.perm, w.seg, pairs, L->top_k, L->hidden, kp_in,
                                   cap_rows, stream))
    return rc;
  if (int rc = b200moe_ep_barrier(ep, epoch + 2, nullptr, stream)) return rc;
  prof_mark(pc, 3, st);
  // Chunk-size hint for the streaming kernel.  Its launchers take chunks one
  // size below the caller's upper bound when they see four or more experts; a
  // rank that holds fewer of a layer with at least four gets the same here (a
  // segment longer than the chunk costs a second pass, nothing else).
  int seg_hint = max_segment;
  if (L->gate.experts < 4 && L->experts >= 4 && max_segment > 16 && max_segment <= 64)
    seg_hint = (max_segment + 1) / 2;
  if (int rc = b200moe_gate_up(recv_x, w.seg2, cap_rows, seg_hint, &L->gate, &L->up, L->activation,
                               regime, kp_mid, w.a, stream))
    return rc;
  prof_mark(pc, 4, st);
  if (int rc = b200moe_down(w.a, w.seg2, cap_rows, seg_hint, &L->down, regime, ksplit, w.dpart, stream))
    return rc;
  prof_mark(pc, 5, st);
  if (int rc = b200moe_ep_return(ep, w.dpart, ksplit, cap_rows, w.seg2, L->hidden, ret_rows, stream))
    return rc;
  if (int rc = b200moe_ep_barrier(ep, epoch + 3, nullptr, stream)) return rc;
  if (tokens > 0)
    if (int rc = launch_combine(ret_y, B200MOE_DT_BF16, 1, pairs, w.inv, w.gates, h, io_dtype, tokens, L, 1,
                                y, io_dtype, st))
      return rc;
  prof_mark(pc, 6, st);
  return B200MOE_OK;
}

int b200moe_set_token_tile(int32_t rows) {
  B200_REQUIRE(rows == 0 || rows == 64 || rows == 128 || rows == 192, "set_token_tile: 0, 64, 128 or 192");
  g_token_tile = rows == 0 ? 192 : rows;
  return B200MOE_OK;
}

int b200moe_set_stream_wide(int32_t mode) {
  B200_REQUIRE(mode >= -1 && mode <= 1, "set_stream_wide: -1 (by layout), 0 or 1");
  set_stream_wide(mode);
  return B200MOE_OK;
}

int b200moe_trace_enable(int on) { return pair_trace_enable(on != 0); }

int b200moe_trace_read(int64_t* out, size_t count) {
  static_assert(sizeof(int64_t) == sizeof(long long), "trace element size");
  return pair_trace_read(reinterpret_cast<long long*>(out), count);
}

int b200moe_profile_enable(int on) {
  if (on && !g_prof.created) {
    for (int c = 0; c < PROF_CALLS; ++c)
      for (int i = 0; i <= PROF_STAGES; ++i) B200_CHECK_CUDA(cudaEventCreate(&g_prof.ev[c][i]));
    g_prof.created = true;
  }
  g_prof.on = on != 0;
  g_prof.used = 0;
  return B200MOE_OK;
}

int b200moe_profile_read(float* ms_out, int32_t* calls_out) {
  B200_REQUIRE(ms_out && calls_out, "profile_read: NULL argument");
  for (int i = 0; i < PROF_STAGES; ++i) ms_out[i] = 0.f;
  for (int c = 0; c < g_prof.used; ++c) {
    B200_CHECK_CUDA(cudaEventSynchronize(g_prof.ev[c][PROF_STAGES]));
    for (int i = 0; i < PROF_STAGES; ++i) {
      float ms = 0.f;
      B200_CHECK_CUDA(cudaEventElapsedTime(&ms, g_prof.ev[c][i], g_prof.ev[c][i + 1]));
      ms_out[i] += ms;
    }
  }
  *calls_out = g_prof.used;
  g_prof.used = 0;
  return B200MOE_OK;
}

}  // extern "C"
