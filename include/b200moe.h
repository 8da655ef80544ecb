/*
 * b200moe — C ABI of the B200 (sm_100a) mixture-of-experts FFN library.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the
 * given CUDA stream (a cudaStream_t passed as void*; NULL = default stream) and
 * returns without synchronising.  Return value: 0 on success, a negative
 * B200MOE_ERR_* code otherwise; b200moe_last_error() gives the message of the
 * calling thread's last failure.  The library never aborts the process and,
 * unless an entry point says otherwise, allocates no device memory: the caller
 * owns every buffer, including the workspace.
 *
 * Each declaration names the piece of sharktank (paths relative to the
 * sharktank project root) whose torch-eager behaviour it replaces.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_ERR_INVALID (-1)     /* bad argument / unsupported shape */
#define B200MOE_ERR_CUDA (-2)        /* a CUDA runtime or driver call failed */
#define B200MOE_ERR_WORKSPACE (-3)   /* workspace too small */
#define B200MOE_ERR_DEVICE (-4)      /* a kernel reported a bounded-wait timeout or a bounds error */

/* Weight layouts.  Q8_0 and Q4_K consume the *planar* planes of sharktank's
 * BlockScaledLayout (types/layouts.py:194-299) and
 * SuperBlockOffsetScaled_4_6_Layout (types/layouts.py:360-530) in place. */
enum {
  B200MOE_LAYOUT_Q8_0 = 0, /* qs: int8 [E,N,K]; d: fp16 [E,N,K/32] */
  B200MOE_LAYOUT_Q4_K = 1, /* qs: u8 [E,N,K/2] (planar nibbles); sub: half2 [E,N,K/32] from b200moe_q4k_prepare */
  B200MOE_LAYOUT_F16 = 2   /* qs: fp16 [E,N,K] dense */
};

enum { B200MOE_ACT_SILU = 0, B200MOE_ACT_GELU = 1 }; /* F.silu | F.gelu (erf) */
enum { B200MOE_DT_F32 = 0, B200MOE_DT_F16 = 1, B200MOE_DT_BF16 = 2 };
enum { B200MOE_REGIME_AUTO = 0, B200MOE_REGIME_STREAM = 1, B200MOE_REGIME_TENSOR = 2,
       B200MOE_REGIME_TENSOR_PAIR = 3 /* tensor kernel on CTA pairs; explicit only */ };

/* One stacked expert weight tensor `ffn_{gate,up,down}_exps.weight`,
 * logical shape [experts, rows, cols] with cols (the reduction dim) innermost
 * (layers/ffn_moe_block.py:32-34). */
typedef struct {
  int32_t layout;
  int32_t experts;
  int32_t rows;
  int32_t cols;
  const void* qs;  /* quantised values (or dense fp16 values) */
  const void* d;   /* Q8_0: per-block fp16 scales; otherwise NULL */
  const void* sub; /* Q4_K: per-sub-block (scale, min) half2 pairs (required);
                      Q8_0: stage-tiled scales from b200moe_q8_prepare or NULL */
} b200moe_weight_t;

/* Parameters of one MoeBlock (layers/mixture_of_experts_block.py:31-62). */
typedef struct {
  int32_t hidden;      /* d */
  int32_t ffn;         /* F */
  int32_t experts;     /* E (<= 64) */
  int32_t top_k;       /* expert_used_count (<= 8) */
  int32_t activation;  /* B200MOE_ACT_* */
  float rms_epsilon;
  const float* ffn_norm_weight;          /* [d]   ffn_norm.weight */
  const float* router_weight;            /* [E,d] ffn_gate_inp.weight */
  const float* router_bias;              /* [E]   ffn_gate_inp.bias or NULL */
  const float* layer_output_norm_weight; /* [d]   layer_output_norm.weight or NULL */
  b200moe_weight_t gate, up, down;
  /* Expert parallelism: this process owns experts [expert_begin, expert_begin+gate.experts). */
  int32_t expert_begin;
} b200moe_layer_t;

const char* b200moe_version(void);
const char* b200moe_last_error(void);

/* Reads and clears the device status word that kernels set; synchronises the
 * stream.  Bits: 1 a bounded wait gave up, 2 an index check failed (the access
 * was skipped), 4 tensor memory could not be obtained, 8 an expert-GEMM operand
 * act(gate)*up was outside the fp16 range and was clipped to +-65504.  Bits 1, 2
 * and 4 make the call return B200MOE_ERR_DEVICE; bit 8 alone is a warning: the
 * call returns B200MOE_OK and *status_out carries it, so that a checkpoint with
 * activation outliers cannot clip unnoticed.  (The normalised activations
 * cannot leave the fp16 range: |x * rsqrt(mean x^2)| <= sqrt(d).)  0 = clean. */
int b200moe_device_status(void* stream, int32_t* status_out);

/* How long the cross-GPU barrier (b200moe_ep_barrier) spins before it gives up,
 * in GPU clock ticks; 0 restores the default of 2^32 ticks (about two seconds).
 * Process-wide, takes effect for launches made after the call.  No reference
 * counterpart.  Meant for tests and for hosts that want to notice a lost peer
 * sooner; too small a value turns ordinary skew between ranks into errors. */
int b200moe_set_wait_limit(int64_t clock_ticks);

/* layout.dequant() of one weight tensor, bit-exact (types/layouts.py:274-290
 * for Q8_0: fp16(d*q) or the exact fp32 product; types/layouts.py:505-517 for
 * Q4_K: fp16 with one rounding per operation).  out: [E,N,K] of out_dtype
 * (B200MOE_DT_F16 or B200MOE_DT_F32; Q4_K in F32 is the fp16 value widened). */
int b200moe_dequant(const b200moe_weight_t* w, int out_dtype, void* out, void* stream);

/* Q4_K: fold the planar 6-bit sub-scale / sub-min planes and the fp16 d / dmin
 * (SuperBlockOffsetScaled_4_6_Layout planes, types/layouts.py:421-470;
 * layout_utils.py:104-113 for the 6-bit combine) into per-sub-block half2
 * (fp16(d*sc), fp16(dmin*m)) — the first two roundings of the reference
 * dequant.  blocks = E*N*K/256; sub_out: half2 [blocks*8]. */
int b200moe_q4k_prepare(const void* d, const void* dmin, const uint8_t* sb_scales_high,
                        const uint8_t* sb_scales_low, const uint8_t* sb_mins_high,
                        const uint8_t* sb_mins_low, int64_t blocks, void* sub_out, void* stream);

/* Q8_0, optional: the block scales `d` [rows, cols/32] (rows = E*N) transposed
 * to [cols/256][rows][8] so that the scales of a 256-k stage are one contiguous
 * run per row tile.  Pass the result as b200moe_weight_t.sub; with sub == NULL
 * the kernels fetch the scales from `d` (slower, no extra memory).
 * sub_out: rows*cols/32 fp16 values. */
int b200moe_q8_prepare(const void* d, int64_t rows, int32_t cols, void* sub_out, void* stream);

/* Packed GGUF blocks -> the planar planes above (types/gguf_interop/layouts.py:
 * 51-60 Q8_0.unpack; :112-153 Q4_K.unpack with _unpack_gguf_i6_scale_mins
 * :163-217).  raw: blocks*34 (Q8_0) or blocks*144 (Q4_K) bytes. */
int b200moe_gguf_unpack_q8_0(const uint8_t* raw, int64_t blocks, void* d_out, int8_t* qs_out,
                             void* stream);
int b200moe_gguf_unpack_q4_k(const uint8_t* raw, int64_t blocks, void* d_out, void* dmin_out,
                             uint8_t* sb_scales_high, uint8_t* sb_scales_low,
                             uint8_t* sb_mins_high, uint8_t* sb_mins_low, uint8_t* qs_out,
                             void* stream);

/* Router: RMSNormLayer (layers/norm.py:34-41, ops/default_impls.py:402-408),
 * ffn_gate_inp linear (ops/default_impls.py:328-341), fp32 softmax, top-k and
 * renormalisation (layers/mixture_of_experts_block.py:66-83).
 * h: [T,d] of h_dtype (F32 or BF16).  Outputs: xn fp16 [T,d] (the normalised
 * activations as expert-GEMM operand), experts int32 [T,k] in descending
 * probability order, gates fp32 [T,k]. */
int b200moe_router(const void* h, int h_dtype, int32_t tokens, const b200moe_layer_t* layer,
                   void* xn_out, int32_t* experts_out, float* gates_out, void* stream);

/* Token permutation (no reference function; definition: pairs p = token*k+slot
 * stably sorted by expert id).  experts: int32 [pairs] with global expert ids;
 * pairs whose expert lies outside [expert_begin, expert_begin+experts_local)
 * are dropped.  counts [E_local], seg_offsets [E_local+1], perm [pairs]
 * (sorted position -> pair), inv [pairs] (pair -> sorted position or -1). */
int b200moe_route_plan(const int32_t* experts, int32_t pairs, int32_t expert_begin,
                       int32_t experts_local, int32_t* counts, int32_t* seg_offsets,
                       int32_t* perm, int32_t* inv, void* stream);

/* Decode front end in one launch: b200moe_router + b200moe_route_plan (all
 * experts local, expert_begin 0) + b200moe_permute_rows, with bit-identical
 * outputs except that the fp16 copy of the normalised rows is not produced.
 * One CTA per token in a cooperative launch; b200moe_front_supported says
 * whether the shape qualifies (at most 128 tokens, hidden <= 8192 and a
 * multiple of 256).  No reference counterpart: the reference runs these steps
 * as separate torch operators (layers/mixture_of_experts_block.py:66-83,
 * layers/ffn_moe_block.py:37-41).  The launch takes one of 32 grid-barrier
 * slots per device in rotation; that host-side rotation is not synchronised
 * between threads: one thread per device issues these calls. */
int b200moe_front_supported(int32_t tokens, const b200moe_layer_t* layer);
int b200moe_front(const void* h, int h_dtype, int32_t tokens, const b200moe_layer_t* layer,
                  int kperm, int32_t* experts_out, float* gates_out, int32_t* counts,
                  int32_t* seg_offsets, int32_t* perm, int32_t* inv, void* xs_out, void* stream);

/* xs[pos,:] = xn[perm[pos] / top_k,:] for pos < seg_offsets[E_local]: the rows
 * each expert multiplies, contiguous per expert (replaces the per-token weight
 * gather `weights[experts]` of layers/ffn_moe_block.py:37-41). */
int b200moe_permute_rows(const void* xn, const int32_t* perm, const int32_t* seg_offsets,
                         int32_t experts_local, int32_t pairs, int32_t top_k, int32_t hidden,
                         int32_t kperm, void* xs_out, void* stream);

/* Whether the expert-GEMM kernels for this weight layout want their input
 * columns in the interleaved order 0,4,1,5,2,6,3,7 within every group of eight
 * (1) or in natural order (0).  Pass the value to b200moe_permute_rows (for the
 * gate/up input) and to b200moe_gate_up (for its output, the down input). */
int b200moe_kperm(int layout, int regime, int32_t max_segment);

/* act(xs W_gate[e]^T) * (xs W_up[e]^T) per expert segment: the "mk,menk->men"
 * einsums of pre_matmul_gather, the activation and the product
 * (layers/ffn_moe_block.py:60-71; ops/default_impls.py:72-81).  xs fp16
 * [pairs,d] sorted rows; a_out fp16 [pairs,F].  max_segment: an upper bound on
 * the rows of any one expert (the token count when experts are not sharded). */
int b200moe_gate_up(const void* xs, const int32_t* seg_offsets, int32_t pairs,
                    int32_t max_segment, const b200moe_weight_t* gate,
                    const b200moe_weight_t* up, int activation, int regime, int32_t out_kperm,
                    void* a_out, void* stream);

/* Number of k-split partial sums the down projection should use.  `pairs` is the
 * number of rows expected (an estimate is fine: it only steers load balance);
 * pass the result to b200moe_down and size d_out with it. */
int b200moe_down_ksplit(const b200moe_weight_t* down, int32_t pairs, int32_t max_segment,
                        int regime);

/* Down projection per expert segment: the "mek,menk->men" einsum
 * (layers/ffn_moe_block.py:70-72; ops/default_impls.py:84-94).  a fp16
 * [pairs,F]; d_out fp32 [ksplit, pairs, d] partial sums with ksplit =
 * b200moe_down_ksplit(...) (the combine adds the partials in index order). */
int b200moe_down(const void* a, const int32_t* seg_offsets, int32_t pairs, int32_t max_segment,
                 const b200moe_weight_t* down, int regime, int32_t ksplit, float* d_out,
                 void* stream);

/* No counterpart in the reference.  The same down projection as b200moe_down
 * for hosts that cannot allocate device memory where they call the layer (an
 * allocator's own callback, a runtime that owns the whole device heap, a decode
 * loop that bans allocator calls): the k-split partial sums live in an 8 MiB
 * array built into the library (held by every GPU that loads it until the
 * process exits) and the caller receives the finished sums.
 * d_out: fp32 [pairs, d]; rows at and after seg_offsets[experts] are set to 0.
 * Always runs the weight-streaming kernel.  Limit: ksplit * pairs * d <=
 * 2,097,152 floats with ksplit = b200moe_down_ksplit(down, pairs, max_segment,
 * B200MOE_REGIME_STREAM) (e.g. 128 pairs at d = 4096); larger calls fail with
 * B200MOE_ERR_INVALID and a message.  Calls no cudaMalloc / cudaFree.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); later calls reuse it.
 * All calls share the one array and nothing in it needs clearing between
 * calls (every partial that is read was written by the same call), but two
 * calls that overlap on the GPU (different streams) race on it.  The host-side
 * lookup of the array's address is not synchronised either: make the first call
 * on a device from one thread before other threads use this entry point. */
int b200moe_down_noalloc(const void* a, const int32_t* seg_offsets, int32_t pairs,
                         int32_t max_segment, const b200moe_weight_t* down, float* d_out,
                         void* stream);

/* y[t] = h[t] + norm?( sum_slot gates[t,slot] * D[inv[t*k+slot]] ): the
 * "me,men->men" scaling and torch.sum over slots (layers/ffn_moe_block.py:
 * 73-74), the optional layer_output_norm and the residual
 * (layers/mixture_of_experts_block.py:86-90).  d_partials: [ksplit, pairs, d]
 * of d_dtype (F32, or BF16 for rows that came back from another rank).  Pairs
 * with inv < 0 contribute nothing.  If add_residual is 0 the result is the
 * un-normalised weighted sum. */
int b200moe_combine(const void* d_partials, int d_dtype, int32_t ksplit, int32_t pairs,
                    const int32_t* inv, const float* gates, const void* h, int h_dtype,
                    int32_t tokens, const b200moe_layer_t* layer, int add_residual, void* y_out,
                    int y_dtype, void* stream);

/* Expert parallelism (no reference counterpart: the reference holds all shards
 * in one process, ops/sharded_impls.py).  Rows arriving from `world` source
 * ranks, each source's rows ordered by local expert, are regrouped per expert:
 * counts[s*experts_local + e] = rows from source s for local expert e;
 * seg_offsets [experts_local+1]; perm [rows] (grouped position -> arrival
 * position); inv [rows] (arrival position -> grouped position). */
int b200moe_exchange_plan(const int32_t* counts, int32_t world, int32_t experts_local,
                          int32_t* seg_offsets, int32_t* perm, int32_t* inv, void* stream);

/* out[i,:] = rows[idx[i] / div,:] for i < n; row_bytes a multiple of 16. */
int b200moe_gather_rows(const void* rows, const int32_t* idx, int32_t n, int32_t div,
                        int32_t row_bytes, void* out, void* stream);

/* Peer-to-peer expert parallelism (no reference counterpart).  All pointer
 * arrays are indexed by rank and hold addresses valid on THIS device: entry
 * [rank] is the local buffer, the others are peer mappings of the same buffer
 * on the other ranks (symmetric allocation).
 *   counts_all  int32 [world][E]   row s = rank s's pair counts per global expert
 *   flags       int32 [world]      barrier flags, zero before the first call
 *   recv_x      fp16  [cap_rows][d] rows routed to this rank's experts
 *   ret_y       bf16  [ret_rows][d] results for this rank's own pairs
 * Sequence per layer on every rank: route + route_plan (all E experts) ->
 * ep_publish_counts -> ep_barrier(epoch, seg2) -> ep_dispatch ->
 * ep_barrier(epoch+1) -> gate_up/down on recv_x with seg2 -> ep_return ->
 * ep_barrier(epoch+2) -> combine on ret_y (bf16) with the route plan's inv.
 * Epochs must increase by one per barrier and be the same on all ranks.  Waits
 * are bounded (about two seconds): a missing peer sets the device status word
 * instead of hanging. */
typedef struct {
  int32_t world, rank, experts_local;
  void* counts_all[16];
  void* flags[16];
  void* recv_x[16];
  void* ret_y[16];
} b200moe_ep_t;

int b200moe_ep_publish_counts(const b200moe_ep_t* ep, const int32_t* counts, void* stream);
/* seg2_out (optional): [experts_local+1] segment offsets of the rows this rank
 * will receive, derived from the completed counts matrix. */
int b200moe_ep_barrier(const b200moe_ep_t* ep, int32_t epoch, int32_t* seg2_out, void* stream);
/* Pushes xn[perm[i]/top_k] for every sorted pair i into the owner's recv_x. */
int b200moe_ep_dispatch(const b200moe_ep_t* ep, const void* xn, const int32_t* experts,
                        const int32_t* perm, const int32_t* seg_offsets, int32_t pairs,
                        int32_t top_k, int32_t hidden, int32_t kperm, int32_t cap_rows,
                        void* stream);
/* Pushes the rows of d_rows (fp32 [ksplit][cap_rows][d], grouped like recv_x)
 * as bf16 into the source ranks' ret_y. */
int b200moe_ep_return(const b200moe_ep_t* ep, const float* d_rows, int32_t ksplit,
                      int32_t cap_rows, const int32_t* seg2, int32_t hidden, int32_t ret_rows,
                      void* stream);

/* The whole expert-parallel layer from one call (no reference counterpart; the
 * layer semantics are MoeBlock.forward, layers/mixture_of_experts_block.py:
 * 64-90): router -> route plan -> publish counts -> barrier -> dispatch ->
 * barrier -> gate/up -> down -> return -> barrier -> combine, all enqueued on
 * `stream` without touching the host in between.  `layer` holds THIS rank's
 * expert shard (gate/up/down with experts_local experts, expert_begin = rank *
 * experts_local, layer->experts = all experts); h, y: this rank's own tokens
 * [tokens, d].  cap_rows / ret_rows are the row capacities of ep->recv_x and
 * ep->ret_y; max_segment bounds the rows any one local expert can receive;
 * ksplit = b200moe_down_ksplit(&layer->down, expected rows, max_segment,
 * regime).  The call uses barrier epochs epoch+1 .. epoch+3: pass 0 first and
 * add 3 per call, identically on every rank, across all layers that share the
 * exchange buffers.  A rank with no tokens still calls (it owns experts).
 * While b200moe_profile_enable is on, the six recorded stages are router | plan +
 * publish + barrier | dispatch + barrier | gate/up | down | return + barrier +
 * combine. */
size_t b200moe_ep_workspace_bytes(const b200moe_layer_t* layer, int32_t tokens, int32_t cap_rows,
                                  int32_t ksplit);
int b200moe_ep_layer_forward(const b200moe_layer_t* layer, const b200moe_ep_t* ep, const void* h,
                             void* y, int io_dtype, int32_t tokens, int regime, int32_t cap_rows,
                             int32_t ret_rows, int32_t max_segment, int32_t ksplit, int32_t epoch,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of workspace b200moe_layer_forward needs for up to `tokens` tokens. */
size_t b200moe_workspace_bytes(const b200moe_layer_t* layer, int32_t tokens);

/* Whole MoeBlock.forward (layers/mixture_of_experts_block.py:64-90) on one
 * device: router -> route plan -> permute -> gate/up -> down -> combine.
 * h, y: [T,d] of io_dtype (F32 or BF16).  experts_out / gates_out may be NULL. */
int b200moe_layer_forward(const b200moe_layer_t* layer, const void* h, void* y, int io_dtype,
                          int32_t tokens, int regime, void* workspace, size_t workspace_bytes,
                          int32_t* experts_out, float* gates_out, void* stream);

/* Same call with host buffers: copies h to the device, runs the layer and
 * copies y back on `stream` (pinned host memory makes the copies asynchronous).
 * dev_io: device scratch of at least 2*T*d*sizeof(io_dtype) bytes. */
int b200moe_layer_forward_host(const b200moe_layer_t* layer, const void* h_host, void* y_host,
                               int io_dtype, int32_t tokens, int regime, void* dev_io,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ---- The attention block that precedes every MoE layer --------------------
 * PagedLlamaAttentionBlock (layers/paged_llama_attention_block.py:26-303) with
 * its paged KV cache (layers/kv_cache.py:222-526).  The projections are plain
 * dense products and stay with the caller (a library GEMM, or the quantized
 * linear of this library); these entry points cover the rest. */

/* Geometry of a PagedKVCache page slab (layers/kv_cache.py:246-277): row `page`
 * of the slab is [blocks][2: K, V][stride][kv_heads][head_dim]. */
typedef struct {
  int32_t blocks;     /* transformer_block_count */
  int32_t stride;     /* block_seq_stride: positions per page */
  int32_t kv_heads;   /* attn_head_count of the cache (kv heads) */
  int32_t head_dim;
  int32_t page_count; /* rows of the slab */
} b200moe_kv_cache_t;

/* RMSNormLayer.forward (layers/norm.py:34-41): y = w * (x * rsqrt(mean(x^2) +
 * eps)) in fp32, x / y [rows, d] of x_dtype / y_dtype (F32, F16 or BF16). */
int b200moe_rms_norm(const void* x, int x_dtype, const float* weight, int64_t rows, int32_t d, float eps,
                     void* y, int y_dtype, void* stream);

/* Rotary embedding of q and k (layers/rotary_embedding.py:115-240 with
 * kernels/templates/rotary_embedding.mlir: pairs (2i, 2i+1), angle position *
 * freqs[i]) fused with the cache write of PagedKVCache.write / write_timestep
 * (layers/kv_cache.py:428-526).  q [tokens, heads, hd] is rotated in place; k is
 * rotated and, like v, stored at its position's slot of page
 * page_ids[seq, position / stride] for transformer block `block_index`; k_out /
 * v_out (both or neither) receive the same rows contiguously (prefill attends
 * them directly).  positions [tokens]: absolute position of every token;
 * tokens_per_seq consecutive tokens belong to one sequence; page_ids [sequences,
 * pages_per_seq]; freqs [hd/2] fp32 = base^-(2i/hd).  A position whose page is
 * missing or out of range sets the bounds bit of the status word and is not
 * written. */
int b200moe_attn_rope_kv_write(void* q, const void* k, const void* v, void* k_out, void* v_out, int io_dtype,
                               void* slab, int cache_dtype, const b200moe_kv_cache_t* cache,
                               int32_t block_index, const int32_t* positions, const int32_t* page_ids,
                               const float* freqs, int32_t tokens, int32_t tokens_per_seq,
                               int32_t pages_per_seq, int32_t heads, void* stream);

/* One decode step of attention over the paged cache: replaces PagedKVCache.read
 * into a linear temporary (layers/kv_cache.py:351-426), the GQA expansion, the
 * decomposed matmul / softcap / mask / fp32 softmax / matmul
 * (paged_llama_attention_block.py:176-214).  K and V rows are read from the pages
 * through page_ids; positions at or beyond seq_lens[seq] are not attended (what
 * the reference's decode mask expresses).  q, out: [bs, heads, hd]; softcap <= 0
 * means none; scratch of b200moe_attn_decode_scratch_bytes(...) bytes holds the
 * partial results of the position splits.  head_dim 64 or 128, heads / kv_heads
 * at most 8. */
size_t b200moe_attn_decode_scratch_bytes(const b200moe_kv_cache_t* cache, int32_t bs, int32_t heads,
                                         int32_t max_seq_len);
int b200moe_attn_decode(const void* q, int q_dtype, const void* slab, int cache_dtype,
                        const b200moe_kv_cache_t* cache, int32_t block_index, const int32_t* page_ids,
                        const int32_t* seq_lens, int32_t bs, int32_t pages_per_seq, int32_t heads,
                        int32_t max_seq_len, float scale, float softcap, void* out, int out_dtype,
                        void* scratch, size_t scratch_bytes, void* stream);

/* A stream of batches from host memory (no reference counterpart: the
 * reference's eager layer takes whatever device its tensors are on).  The
 * pipeline keeps `depth` steps in flight: the host->device copy of a step's
 * input, the layer, and the device->host copy of its output run on three
 * streams linked by events, so consecutive steps overlap and the sustained rate
 * is the layer's own as long as a copy is shorter than the layer.  Pinned host
 * buffers are required for the copies to be asynchronous.
 *   b200moe_pipeline_bytes   device memory the caller must provide (2*depth
 *                            activation buffers of max_tokens rows + the workspace)
 *   b200moe_pipeline_create  builds the pipeline on the current device; creates
 *                            two streams and 3*depth events, allocates no
 *                            device memory; the layer descriptor is copied
 *   b200moe_pipeline_submit  enqueues one step (h_host -> layer -> y_host); the
 *                            layer runs on `stream`.  Returns without waiting,
 *                            except that it first waits for the output copy of
 *                            the step that used the same slot `depth` submits
 *                            ago.  y_host is complete after a later submit has
 *                            reused its slot or after b200moe_pipeline_drain.
 *                            h_host / y_host must stay untouched until then.
 *   b200moe_pipeline_drain   waits for every submitted step's output copy
 *   b200moe_pipeline_destroy drains, then frees the streams and events
 * Not thread-safe: one thread drives one pipeline. */
typedef struct b200moe_pipeline b200moe_pipeline_t;
size_t b200moe_pipeline_bytes(const b200moe_layer_t* layer, int io_dtype, int32_t max_tokens,
                              int32_t depth);
int b200moe_pipeline_create(const b200moe_layer_t* layer, int io_dtype, int32_t max_tokens,
                            int regime, int32_t depth, void* dev_mem, size_t dev_bytes,
                            b200moe_pipeline_t** out);
int b200moe_pipeline_submit(b200moe_pipeline_t* p, const void* h_host, void* y_host,
                            int32_t tokens, void* stream);
int b200moe_pipeline_drain(b200moe_pipeline_t* p);
int b200moe_pipeline_destroy(b200moe_pipeline_t* p);

/* Stage timing for benchmarks (no reference counterpart).  While enabled,
 * b200moe_layer_forward brackets each of its six stages (router, route plan,
 * permute, gate/up, down, combine) with CUDA events on the call's stream; up to
 * 512 calls are kept.  b200moe_profile_read synchronises those events, adds the
 * per-stage milliseconds of all recorded calls into ms_out[6], returns the
 * number of calls through *calls_out and clears the record. */
int b200moe_profile_enable(int on);
int b200moe_profile_read(float* ms_out, int32_t* calls_out);

/* Tuning knob (no reference counterpart): upper bound of the single-CTA tensor
 * kernel's token tile, 64, 128 or 192 rows (0 restores the default, 192).
 * Narrower tiles leave more tensor memory for staged weights (6 / 4 / 2 slots)
 * and re-stream the weights once per tile.  Process-wide; results do not depend
 * on it beyond fp32 summation inside a tile being unchanged (bit-identical). */
int b200moe_set_token_tile(int32_t rows);

/* Tuning knob (no reference counterpart): warp geometry of the streaming kernel
 * for chunks of up to 32 tokens.  1 = sixteen consumer warps per CTA (each stage's
 * reduction range split four ways), 0 = eight, -1 (default) = sixteen for the
 * quantised layouts, eight for dense fp16 weights.
 * Process-wide.  The fp32 summation order inside a stage differs between the two
 * geometries, so results agree to rounding, not bit for bit. */
int b200moe_set_stream_wide(int32_t mode);

/* Diagnostic (no reference counterpart): while enabled, every launch of the
 * CTA-pair tensor kernel records clock64 time stamps of its first CTA pair's
 * warp roles for the first 256 stages.  b200moe_trace_read synchronises the
 * device and copies the last launch's record: int64 [2 CTAs][5 roles][256
 * stages][8 points]; roles: 0 weight producer (0 before / 1 after its wait for
 * a free slot), 1 token producer (0 / 1 likewise), 2 MMA issuer (0 start, 1
 * tokens arrived, 2 A operand ready, 3 MMAs issued), 3 and 4 the two dequant
 * groups (0 start, 1 weights arrived, 2 dequantised, 3 A slot free, 4 stored).
 * clock64 counts per SM: the two CTAs' stamps are not on one time base.
 * count = number of int64 values `out` can hold (at least 20480). */
int b200moe_trace_enable(int on);
int b200moe_trace_read(int64_t* out, size_t count);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
