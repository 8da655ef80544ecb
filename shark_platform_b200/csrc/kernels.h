// Launchers implemented by the kernel translation units; called by the C ABI.
#pragma once
#include "common.cuh"

namespace b200moe {

int launch_router(const void* h, int h_dtype, int tokens, const b200moe_layer_t* L, void* xn,
                  int32_t* experts, float* gates, cudaStream_t st);
int launch_route_plan(const int32_t* experts, int pairs, int e_begin, int E, int32_t* counts,
                      int32_t* seg, int32_t* perm, int32_t* inv, cudaStream_t st);
int launch_permute_rows(const void* xn, const int32_t* perm, const int32_t* seg, int E, int pairs,
                        int k, int d, int kperm, void* xs, cudaStream_t st);
// router + route plan + permutation in one cooperative launch (small token counts)
bool front_fused_supported(int tokens, const b200moe_layer_t* L);
int launch_front_fused(const void* h, int h_dtype, int tokens, const b200moe_layer_t* L,
                       int32_t* experts, float* gates, int32_t* counts, int32_t* seg,
                       int32_t* perm, int32_t* inv, int kperm, void* xs, int32_t* status,
                       cudaStream_t st);
int clear_front_sync(cudaStream_t st);
int launch_exchange_plan(const int32_t* counts, int world, int el, int32_t* seg, int32_t* perm,
                         int32_t* inv, cudaStream_t st);
int launch_gather_rows(const void* rows, const int32_t* idx, int n, int div, int row_bytes,
                       void* out, cudaStream_t st);
int launch_combine(const void* dpart, int d_dtype, int ksplit, int pairs, const int32_t* inv,
                   const float* gates, const void* h, int h_dtype, int tokens,
                   const b200moe_layer_t* L, int add_residual, void* y, int y_dtype,
                   cudaStream_t st);
int launch_dequant(const b200moe_weight_t* w, int out_dtype, void* out, cudaStream_t st);
int launch_q4k_prepare(const void* d, const void* dmin, const uint8_t* sh, const uint8_t* sl,
                       const uint8_t* mh, const uint8_t* ml, long long blocks, void* sub,
                       cudaStream_t st);
int launch_q8_prepare(const void* d, long long rows, int cols, void* out, cudaStream_t st);
int launch_gguf_q8(const uint8_t* raw, long long blocks, void* d, int8_t* qs, cudaStream_t st);
int launch_gguf_q4k(const uint8_t* raw, long long blocks, void* d, void* dmin, uint8_t* sh,
                    uint8_t* sl, uint8_t* mh, uint8_t* ml, uint8_t* qs, cudaStream_t st);

// decode regime (stream_gemm.cu)
int stream_down_ksplit(const b200moe_weight_t* down, int pairs);
int launch_stream_gate_up(const void* xs, const int32_t* seg, int pairs, int max_segment,
                          const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                          int out_kperm, void* a_out, cudaStream_t st);
int launch_stream_down(const void* a_in, const int32_t* seg, int pairs, int max_segment,
                       const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st);
// -1 = wide geometry (16 consumer warps) by layout, 0 = never, 1 = always
void set_stream_wide(int mode);

// prefill regime (tc_gemm.cu)
bool tc_supported(const b200moe_weight_t* w, bool down);
int launch_tc_gate_up(const void* xs, const int32_t* seg, int pairs, int tok_tile,
                      const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                      int out_kperm, void* a_out, cudaStream_t st);
int tc_down_ksplit(const b200moe_weight_t* down, int est_pairs);
int launch_tc_down(const void* a_in, const int32_t* seg, int pairs, int tok_tile,
                   const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st);

// prefill regime on CTA pairs (tc_pair_gemm.cu)
bool tc_pair_supported_gate_up(const b200moe_weight_t* gate);
bool tc_pair_supported_down(const b200moe_weight_t* down);
int launch_tc_pair_gate_up(const void* xs, const int32_t* seg, int pairs, int tok_tile,
                           const b200moe_weight_t* gate, const b200moe_weight_t* up, int act,
                           int out_kperm, void* a_out, cudaStream_t st);
int launch_tc_pair_down(const void* a_in, const int32_t* seg, int pairs, int tok_tile,
                        const b200moe_weight_t* down, int ksplit, float* d_out, cudaStream_t st);

int pair_trace_enable(bool on);
int pair_trace_read(long long* out, size_t count);

}  // namespace b200moe
