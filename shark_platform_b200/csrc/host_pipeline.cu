// Host-buffer pipeline around the layer call: step n+1's host->device copy and
// step n-1's device->host copy run on their own streams while step n's kernels
// run, so a stream of batches from pinned host memory costs the layer time,
// not layer time plus two PCIe transfers.
//
// Per slot (ring of `depth` slots): an input and an output buffer on the
// device, three events.  The layer workspace is shared by all slots: the layer
// calls themselves are serialised on the caller's stream.
//   copy-in stream : h_host -> h_dev[slot]                     record in_done[slot]
//   caller's stream: wait in_done[slot]; layer; record comp_done[slot]
//   copy-out stream: wait comp_done[slot]; y_dev[slot] -> y_host; record out_done[slot]
// A slot is reused only after the host has waited for its out_done event, which
// also means that y_host of that earlier step is complete.
#include <new>

#include "kernels.h"

struct b200moe_pipeline {
  b200moe_layer_t layer;
  int io_dtype, regime, depth, max_tokens, device;
  size_t io_bytes;         // bytes of one [max_tokens, hidden] buffer, 1 KiB aligned
  size_t workspace_bytes;
  uint8_t* dev_mem;        // [depth][2][io_bytes] then the workspace
  cudaStream_t s_in, s_out;
  cudaEvent_t in_done[8], comp_done[8], out_done[8];
  bool busy[8];
  long long submitted;
};

using namespace b200moe;

namespace {
constexpr int PIPE_MAX_DEPTH = 8;
inline size_t up1k(size_t v) { return (v + 1023) / 1024 * 1024; }
inline size_t elem_bytes(int dt) { return dt == B200MOE_DT_F32 ? 4 : 2; }
}  // namespace

extern "C" {

size_t b200moe_pipeline_bytes(const b200moe_layer_t* layer, int io_dtype, int32_t max_tokens,
                              int32_t depth) {
  if (layer == nullptr || max_tokens <= 0 || depth < 1 || depth > PIPE_MAX_DEPTH) return 0;
  const size_t io = up1k(static_cast<size_t>(max_tokens) * layer->hidden * elem_bytes(io_dtype));
  return 2 * io * depth + up1k(b200moe_workspace_bytes(layer, max_tokens));
}

int b200moe_pipeline_create(const b200moe_layer_t* layer, int io_dtype, int32_t max_tokens,
                            int regime, int32_t depth, void* dev_mem, size_t dev_bytes,
                            b200moe_pipeline_t** out) {
  B200_REQUIRE(layer && out && dev_mem, "pipeline_create: NULL argument");
  B200_REQUIRE(io_dtype == B200MOE_DT_F32 || io_dtype == B200MOE_DT_BF16,
               "pipeline_create: activations must be fp32 or bf16");
  B200_REQUIRE(max_tokens > 0 && depth >= 1 && depth <= PIPE_MAX_DEPTH,
               "pipeline_create: max_tokens must be positive and depth 1..%d", PIPE_MAX_DEPTH);
  const size_t need = b200moe_pipeline_bytes(layer, io_dtype, max_tokens, depth);
  if (dev_bytes < need) {
    set_error("pipeline_create: needs %zu bytes of device memory, got %zu", need, dev_bytes);
    return B200MOE_ERR_WORKSPACE;
  }
  b200moe_pipeline* p = new (std::nothrow) b200moe_pipeline();
  B200_REQUIRE(p != nullptr, "pipeline_create: out of host memory");
  p->layer = *layer;
  p->io_dtype = io_dtype; p->regime = regime; p->depth = depth; p->max_tokens = max_tokens;
  p->io_bytes = up1k(static_cast<size_t>(max_tokens) * layer->hidden * elem_bytes(io_dtype));
  p->workspace_bytes = b200moe_workspace_bytes(layer, max_tokens);
  p->dev_mem = static_cast<uint8_t*>(dev_mem);
  p->submitted = 0;
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking);
  for (int i = 0; i < depth && e == cudaSuccess; ++i) {
    p->busy[i] = false;
    e = cudaEventCreateWithFlags(&p->in_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->comp_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->out_done[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    delete p;
    return cuda_fail(e, "pipeline_create: streams/events");
  }
  *out = p;
  return B200MOE_OK;
}

int b200moe_pipeline_submit(b200moe_pipeline_t* p, const void* h_host, void* y_host,
                            int32_t tokens, void* stream) {
  B200_REQUIRE(p && h_host && y_host, "pipeline_submit: NULL argument");
  B200_REQUIRE(tokens > 0 && tokens <= p->max_tokens, "pipeline_submit: %d tokens, pipeline holds %d",
               tokens, p->max_tokens);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int slot = static_cast<int>(p->submitted % p->depth);
  if (p->busy[slot]) B200_CHECK_CUDA(cudaEventSynchronize(p->out_done[slot]));
  const size_t bytes = static_cast<size_t>(tokens) * p->layer.hidden * elem_bytes(p->io_dtype);
  uint8_t* dh = p->dev_mem + static_cast<size_t>(slot) * 2 * p->io_bytes;
  uint8_t* dy = dh + p->io_bytes;
  uint8_t* ws = p->dev_mem + static_cast<size_t>(p->depth) * 2 * p->io_bytes;
  B200_CHECK_CUDA(cudaMemcpyAsync(dh, h_host, bytes, cudaMemcpyHostToDevice, p->s_in));
  B200_CHECK_CUDA(cudaEventRecord(p->in_done[slot], p->s_in));
  B200_CHECK_CUDA(cudaStreamWaitEvent(st, p->in_done[slot], 0));
  if (int rc = b200moe_layer_forward(&p->layer, dh, dy, p->io_dtype, tokens, p->regime, ws,
                                     p->workspace_bytes, nullptr, nullptr, stream))
    return rc;
  B200_CHECK_CUDA(cudaEventRecord(p->comp_done[slot], st));
  B200_CHECK_CUDA(cudaStreamWaitEvent(p->s_out, p->comp_done[slot], 0));
  B200_CHECK_CUDA(cudaMemcpyAsync(y_host, dy, bytes, cudaMemcpyDeviceToHost, p->s_out));
  B200_CHECK_CUDA(cudaEventRecord(p->out_done[slot], p->s_out));
  p->busy[slot] = true;
  p->submitted++;
  return B200MOE_OK;
}

int b200moe_pipeline_drain(b200moe_pipeline_t* p) {
  B200_REQUIRE(p != nullptr, "pipeline_drain: NULL pipeline");
  for (int i = 0; i < p->depth; ++i) {
    if (p->busy[i]) {
      B200_CHECK_CUDA(cudaEventSynchronize(p->out_done[i]));
      p->busy[i] = false;
    }
  }
  return B200MOE_OK;
}

int b200moe_pipeline_destroy(b200moe_pipeline_t* p) {
  if (p == nullptr) return B200MOE_OK;
  int rc = b200moe_pipeline_drain(p);
  for (int i = 0; i < p->depth; ++i) {
    cudaEventDestroy(p->in_done[i]);
    cudaEventDestroy(p->comp_done[i]);
    cudaEventDestroy(p->out_done[i]);
  }
  cudaStreamDestroy(p->s_in);
  cudaStreamDestroy(p->s_out);
  delete p;
  return rc;
}

}  // extern "C"
