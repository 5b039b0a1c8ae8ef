// Graph / tape host logic: see graph.h.  Every op follows the shape rules of its reference
// counterpart (cited per op) and launches kernels of this library on the graph's stream; there
// is no host synchronisation inside an op and no per-op cudaMalloc once the pool is warm.
#include "graph.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "../../../include/eisen_b200.h"

namespace eisen {

namespace {

inline size_t dsize(int dt) { return dt == 1 ? 2 : 4; }
inline int64_t numel_of(const std::vector<int64_t>& s) {
  int64_t n = 1;
  for (int64_t d : s) n *= d;
  return n;
}
inline size_t round256(size_t b) { return (b + 255) & ~size_t(255); }

void ck(int rc, const char* what) {
  if (rc != 0) throw EisenException(rc, std::string(what) + ": " + eisen_last_error());
}
void cuck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw EisenException(EISEN_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
[[noreturn]] void invalid(const std::string& m) { throw EisenException(EISEN_ERR_INVALID, m); }

}  // namespace

// ------------------------------------------------------------------------------------- storage
namespace {
size_t env_mb(const char* name, size_t fallback_mb) {
  const char* v = std::getenv(name);
  if (!v || !*v) return fallback_mb;
  char* end = nullptr;
  const unsigned long long mb = std::strtoull(v, &end, 10);
  return (end && *end == 0) ? (size_t)mb : fallback_mb;
}
void* host_alloc(size_t bytes) {
  void* p = nullptr;
  cuck(cudaHostAlloc(&p, std::max<size_t>(bytes, 16), cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc");
  void* d = nullptr;
  cuck(cudaHostGetDevicePointer(&d, p, 0), "cudaHostGetDevicePointer");
  if (d != p) {
    cudaFreeHost(p);
    throw EisenException(EISEN_ERR_CUDA, "host-homed parameters need unified addressing (host and device pointer differ)");
  }
  return p;
}
}  // namespace

Graph::Graph(Precision prec, cudaStream_t s) : precision(prec), stream(s) {
  // src/graph/mod.rs:283-288
  vram_budget_bytes = env_mb("EISEN_VRAM_BUDGET_MB", 0) << 20;
  activation_reserve_bytes = env_mb("EISEN_ACTIVATION_RESERVE_MB", 64) << 20;
  cuck(cudaMalloc(&status_dev, 256), "cudaMalloc(status)");
  cuck(cudaMemsetAsync(status_dev, 0, 256, stream), "memset(status)");
  bad_id_dev = status_dev + 16;
}

Graph::~Graph() {
  cudaStreamSynchronize(stream);
  for (HTensor& t : tensors) free_tensor(t);
  for (auto& kv : pool_)
    for (void* p : kv.second) cudaFree(p);
  for (auto& kv : rope_tables_) cudaFree(kv.second);
  if (scratch_) cudaFree(scratch_);
  if (arena_w) cudaFree(arena_w);
  if (arena_shadow) cudaFree(arena_shadow);
  if (arena_g) cudaFree(arena_g);
  if (status_dev) cudaFree(status_dev);
  for (StageSlot& sl : stage_) {
    if (sl.buf) cudaFree(sl.buf);
    if (sl.ready) cudaEventDestroy(sl.ready);
  }
  if (compute_mark_) cudaEventDestroy(compute_mark_);
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
  if (aux_stream_) cudaStreamDestroy(aux_stream_);
  if (aux_fork_) cudaEventDestroy(aux_fork_);
  if (aux_join_) cudaEventDestroy(aux_join_);
}

// exact-size free lists, as the reference's vram_pool keyed by element count
// (src/graph/mod.rs:62-64, 437-556)
void* Graph::pool_get(size_t bytes) {
  bytes = round256(std::max<size_t>(bytes, 4));
  auto it = pool_.find(bytes);
  if (it != pool_.end() && !it->second.empty()) {
    void* p = it->second.back();
    it->second.pop_back();
    pool_bytes_cached -= bytes;
    pool_bytes_live += bytes;
    ++pool_hits;
    return p;
  }
  // src/graph/memory.rs:189-266 (safe_alloc_zeros): allocate if the budget allows; else drop the
  // cached pool buffers and try again; else fail (with a status, where the reference panics)
  if (capturing)
    throw EisenException(EISEN_ERR_INVALID, "a pooled buffer of " + std::to_string(bytes) + " bytes is not cached: run the step "
                                                "once before capturing it, so that the capture allocates nothing");
  auto within_budget = [&]() { return vram_budget_bytes == 0 || current_vram_usage() + bytes <= vram_budget_bytes; };
  void* p = nullptr;
  cudaError_t e = within_budget() ? cudaMalloc(&p, bytes) : cudaErrorMemoryAllocation;
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaStreamSynchronize(stream);
    for (auto& kv : pool_) {
      for (void* q : kv.second) cudaFree(q);
      kv.second.clear();
    }
    device_bytes_allocated -= pool_bytes_cached;
    pool_bytes_cached = 0;
    if (!within_budget())
      throw EisenException(EISEN_ERR_OOM, "VRAM budget exhausted: " + std::to_string(current_vram_usage() >> 20) + " MB in use, " +
                                              std::to_string(bytes >> 20) + " MB requested, budget " +
                                              std::to_string(vram_budget_bytes >> 20) + " MB");
    e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) throw EisenException(EISEN_ERR_OOM, "out of device memory in the activation pool");
  }
  device_bytes_allocated += bytes;
  pool_bytes_live += bytes;
  ++pool_misses;
  return p;
}

void Graph::pool_put(void* p, size_t bytes) {
  if (!p) return;
  bytes = round256(std::max<size_t>(bytes, 4));
  pool_[bytes].push_back(p);
  pool_bytes_cached += bytes;
  pool_bytes_live -= bytes;
}

void* Graph::scratch(size_t bytes) {
  if (bytes > scratch_bytes_) {
    // the old buffer may still be in use by queued kernels: hand it to the pool instead of freeing
    if (scratch_) { pool_bytes_live += round256(scratch_bytes_); pool_put(scratch_, scratch_bytes_); }
    scratch_bytes_ = round256(bytes + bytes / 4);
    cuck(cudaMalloc(&scratch_, scratch_bytes_), "cudaMalloc(scratch)");
    device_bytes_allocated += scratch_bytes_;
  }
  return scratch_;
}

int64_t Graph::new_tensor(HTensor&& t) {
  tensors.push_back(std::move(t));
  return (int64_t)tensors.size() - 1;
}

void Graph::free_tensor(HTensor& t) {
  if (t.is_pooled) {
    if (!t.data_kept) pool_put(t.data, (size_t)t.numel * dsize(t.dtype == DT_I32 ? 0 : t.dtype));
    pool_put(t.grad, (size_t)t.numel * dsize(t.grad_dtype));
  } else if (t.host_homed) {
    if (t.data) cudaFreeHost(t.data);
    if (t.shadow) cudaFreeHost(t.shadow);
    if (t.grad) cudaFreeHost(t.grad);
  } else {
    if (t.owns_data && t.data) cudaFree(t.data);
    if (t.owns_data && t.shadow) cudaFree(t.shadow);
    if (t.owns_grad && t.grad) cudaFree(t.grad);
  }
  t.data = t.shadow = t.grad = nullptr;
}

void Graph::reserve_param_arena(int64_t total_elems) {
  if (arena_w) invalid("reserve_param_arena: arena already reserved");
  arena_cap = (total_elems + 63) / 64 * 64;
  cuck(cudaMalloc(&arena_w, (size_t)arena_cap * 4), "cudaMalloc(param arena)");
  cuck(cudaMalloc(&arena_g, (size_t)arena_cap * 4), "cudaMalloc(grad arena)");
  cuck(cudaMemsetAsync(arena_w, 0, (size_t)arena_cap * 4, stream), "memset");
  cuck(cudaMemsetAsync(arena_g, 0, (size_t)arena_cap * 4, stream), "memset");
  if (precision == Precision::Bf16Mixed) {
    cuck(cudaMalloc(&arena_shadow, (size_t)arena_cap * 2), "cudaMalloc(shadow arena)");
    cuck(cudaMemsetAsync(arena_shadow, 0, (size_t)arena_cap * 2, stream), "memset");
  }
  device_bytes_allocated += (size_t)arena_cap * (precision == Precision::Bf16Mixed ? 10 : 8);
}

// src/graph/mod.rs `alloc`: a leaf with host data and a zero gradient.  Leaves created before
// mark_params() are parameters (f32 master data, f32 gradient, bf16 shadow in Bf16Mixed);
// later leaves are inputs (their gradient has the activation dtype).
int64_t Graph::alloc(const std::vector<int64_t>& shape, const float* host) {
  HTensor t;
  t.shape = shape;
  t.numel = numel_of(shape);
  t.dtype = 0;
  const bool param = (num_params == 0);
  t.is_param = param;
  const size_t n = (size_t)std::max<int64_t>(t.numel, 1);
  const int64_t padded = (t.numel + 63) / 64 * 64;
  const bool in_arena = param && !home_params_on_host && arena_w && arena_used + padded <= arena_cap;
  if (param && home_params_on_host) {
    t.data = host_alloc(n * 4);
    t.grad = host_alloc(n * 4);
    t.grad_dtype = 0;
    std::memset(t.grad, 0, n * 4);
    if (precision == Precision::Bf16Mixed) t.shadow = host_alloc(n * 2);
    t.host_homed = true;
  } else if (in_arena) {
    t.data = arena_w + arena_used;
    t.grad = arena_g + arena_used;
    t.grad_dtype = 0;
    if (arena_shadow) t.shadow = static_cast<uint16_t*>(arena_shadow) + arena_used;
    arena_used += padded;
  } else {
    cuck(cudaMalloc(&t.data, round256(n * 4)), "cudaMalloc(leaf)");
    t.owns_data = true;
    t.grad_dtype = param ? 0 : act_dtype();
    cuck(cudaMalloc(&t.grad, round256(n * dsize(t.grad_dtype))), "cudaMalloc(leaf grad)");
    t.owns_grad = true;
    cuck(cudaMemsetAsync(t.grad, 0, n * dsize(t.grad_dtype), stream), "memset(leaf grad)");
    if (precision == Precision::Bf16Mixed) cuck(cudaMalloc(&t.shadow, round256(n * 2)), "cudaMalloc(leaf shadow)");
    device_bytes_allocated += round256(n * 4) * 2;
  }
  t.grad_init = true;  // zero-initialised: every writer accumulates
  int64_t id = new_tensor(std::move(t));
  if (host) load_tensor_data(id, host, tensors[id].numel);
  return id;
}

// token ids as device int32 (the reference keeps them in an f32 tensor, tests/phase2_embedding.rs:16-17)
int64_t Graph::alloc_ids(const std::vector<int64_t>& shape, const int32_t* host_ids, bool async_pinned) {
  HTensor t;
  t.shape = shape;
  t.numel = numel_of(shape);
  t.dtype = DT_I32;
  t.constant = true;
  t.is_pooled = true;
  t.data = pool_get((size_t)t.numel * 4);
  // stream-ordered copy; for pageable memory the runtime stages the source before returning, so
  // the caller's buffer may be reused at once either way
  (void)async_pinned;
  cuck(cudaMemcpyAsync(t.data, host_ids, (size_t)t.numel * 4, cudaMemcpyHostToDevice, stream), "H2D(ids)");
  return new_tensor(std::move(t));
}

int64_t Graph::alloc_pooled_dtype(const std::vector<int64_t>& shape, int dtype) {
  HTensor t;
  t.shape = shape;
  t.numel = numel_of(shape);
  t.dtype = dtype;
  t.grad_dtype = dtype;
  t.is_pooled = true;
  t.data = pool_get((size_t)std::max<int64_t>(t.numel, 1) * dsize(dtype));
  return new_tensor(std::move(t));
}
int64_t Graph::alloc_pooled(const std::vector<int64_t>& shape) { return alloc_pooled_dtype(shape, act_dtype()); }

// src/graph/mod.rs:368-430.  bf16 copies are rounded to nearest (the reference truncates on the
// host, src/tensor.rs:7-9; not reproduced).
void Graph::load_tensor_data(int64_t id, const float* host, int64_t n) {
  HTensor& t = tensors.at(id);
  if (n != t.numel) invalid("load_tensor_data: element count does not match the tensor shape");
  if (t.dtype == 0) {
    cuck(cudaMemcpyAsync(t.data, host, (size_t)n * 4, cudaMemcpyDefault, stream), "H2D");
    if (t.shadow) ck(eisen_cast(stream, t.data, 0, t.shadow, 1, n), "cast(shadow)");
    if (t.host_homed) invalidate_staged_weights();
    cuck(cudaStreamSynchronize(stream), "sync");
  } else if (t.dtype == 1) {
    float* tmp = static_cast<float*>(pool_get((size_t)n * 4));
    cuck(cudaMemcpyAsync(tmp, host, (size_t)n * 4, cudaMemcpyHostToDevice, stream), "H2D");
    ck(eisen_cast(stream, tmp, 0, t.data, 1, n), "cast");
    cuck(cudaStreamSynchronize(stream), "sync");
    pool_put(tmp, (size_t)n * 4);
  } else {
    invalid("load_tensor_data: id tensors are loaded with alloc_ids");
  }
}

static void read_back(Graph& g, const void* dev, int dt, int64_t n, float* out) {
  if (dt == 0) {
    cuck(cudaMemcpyAsync(out, dev, (size_t)n * 4, cudaMemcpyDefault, g.stream), "D2H");
    cuck(cudaStreamSynchronize(g.stream), "sync");
  } else {
    float* tmp = static_cast<float*>(g.pool_get((size_t)n * 4));
    ck(eisen_cast(g.stream, dev, 1, tmp, 0, n), "cast");
    cuck(cudaMemcpyAsync(out, tmp, (size_t)n * 4, cudaMemcpyDeviceToHost, g.stream), "D2H");
    cuck(cudaStreamSynchronize(g.stream), "sync");
    g.pool_put(tmp, (size_t)n * 4);
  }
  g.check_status();
}

void Graph::sync_to_cpu(int64_t id, float* out) {
  HTensor& t = tensors.at(id);
  if (t.dtype == DT_I32) invalid("sync_to_cpu: id tensor");
  read_back(*this, t.data, t.dtype, t.numel, out);
}
void Graph::sync_grad_to_cpu(int64_t id, float* out) {
  HTensor& t = tensors.at(id);
  if (!t.grad || !t.grad_init) {
    std::fill(out, out + t.numel, 0.0f);
    return;
  }
  read_back(*this, t.grad, t.grad_dtype, t.numel, out);
}

void Graph::synchronize() {
  cuck(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  check_status();
}

namespace {
struct CapturedStep {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};
}  // namespace

void Graph::capture_begin() {
  if (capturing) invalid("capture_begin: a capture is already running on this graph");
  cuck(cudaStreamSynchronize(stream), "sync");
  check_status();
  cuck(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
  capturing = true;
}

void* Graph::capture_end() {
  if (!capturing) invalid("capture_end: no capture is running");
  capturing = false;
  CapturedStep* cs = new CapturedStep();
  cudaError_t e = cudaStreamEndCapture(stream, &cs->graph);
  if (e != cudaSuccess || !cs->graph) {
    delete cs;
    cudaGetLastError();
    throw EisenException(EISEN_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e) +
                                             " (the captured step allocated, synchronised or waited on the host?)");
  }
  e = cudaGraphInstantiate(&cs->exec, cs->graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(cs->graph);
    delete cs;
    throw EisenException(EISEN_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
  }
  return cs;
}

void Graph::check_status() {
  int h[32] = {0};
  cuck(cudaMemcpy(h, status_dev, sizeof(h), cudaMemcpyDeviceToHost), "read status");
  if (h[0] != 0) {
    cudaMemset(status_dev, 0, 4);
    throw EisenException(EISEN_ERR_KERNEL, "a tensor-core kernel gave up on a bounded wait (fault code " + std::to_string(h[0]) + ")");
  }
  if (h[16] != 0) {
    cudaMemset(bad_id_dev, 0, 4);
    throw EisenException(EISEN_ERR_INVALID, "gather: a token id is outside [0, vocab)");
  }
  if (h[17] != 0) {
    cudaMemset(bad_id_dev + 1, 0, 4);
    throw EisenException(EISEN_ERR_INVALID, "cross_entropy: a target is neither the ignore index nor inside [0, vocab)");
  }
}

void Graph::release_attn_stash() {
  for (AttnStash& st : attn_stash) {
    // a stashed buffer was never returned to the pool, so it still counts as live: pool_put settles that
    if (st.o) pool_put(st.o, st.o_bytes);
    if (st.o_lo) pool_put(st.o_lo, st.o_bytes);
    if (st.lse) pool_put(st.lse, st.lse_bytes);
    st = AttnStash();
  }
}

void Graph::restore_save_point(int64_t sp) {
  while ((int64_t)tensors.size() > sp) {
    free_tensor(tensors.back());
    tensors.pop_back();
  }
}
void Graph::clear_activations() {
  tape.clear();
  if (aux_pending_ && !capturing) {
    // a forward pass whose backward never ran: its side-stream work still owns a pooled buffer
    cuck(cudaStreamWaitEvent(stream, aux_join_, 0), "cudaStreamWaitEvent");
    aux_pending_ = false;
  }
  restore_save_point(num_params);
}
void Graph::reinterpret_shape(int64_t id, const std::vector<int64_t>& shape) {
  HTensor& t = tensors.at(id);
  if (numel_of(shape) != t.numel) invalid("reinterpret_shape: element count changes");
  t.shape = shape;
}
void Graph::zero_grad(int64_t id) {
  HTensor& t = tensors.at(id);
  if (t.grad) {
    cuck(cudaMemsetAsync(t.grad, 0, (size_t)t.numel * dsize(t.grad_dtype), stream), "memset(grad)");
    t.grad_init = true;
  }
}

void Graph::ensure_grad(int64_t id) {
  HTensor& t = tensors.at(id);
  if (t.grad) return;
  if (t.constant) invalid("ensure_grad: constant tensor");
  t.grad = pool_get((size_t)std::max<int64_t>(t.numel, 1) * dsize(t.grad_dtype));
  t.grad_init = false;
  if (!t.is_pooled) t.owns_grad = false;  // returned through the pool only for pooled tensors
}

void Graph::seed_grad_ones(int64_t id) {
  ensure_grad(id);
  HTensor& t = tensors.at(id);
  if (t.grad_dtype == 0) {
    ck(eisen_fill_f32(stream, static_cast<float*>(t.grad), 1.0f, t.numel), "fill");
  } else {
    float* tmp = static_cast<float*>(pool_get((size_t)t.numel * 4));
    ck(eisen_fill_f32(stream, tmp, 1.0f, t.numel), "fill");
    ck(eisen_cast(stream, tmp, 0, t.grad, 1, t.numel), "cast");
    pool_put(tmp, (size_t)t.numel * 4);  // stream-ordered reuse
  }
  t.grad_init = true;
  t.grad_is_ones = true;
}

// src/graph/mod.rs:670-796: seed with ones, walk the tape in reverse, keep the nodes
void Graph::backward(int64_t loss_id) {
  if (no_grad) return;
  seed_grad_ones(loss_id);
  backward_from(0);
}
void Graph::backward_from(int64_t begin) {
  for (int64_t i = (int64_t)tape.size(); i-- > begin;) tape[i].backward();
}

const void* Graph::operand(const HTensor& t) const {
  if (precision == Precision::Bf16Mixed && t.dtype == 0) {
    if (!t.shadow) throw EisenException(EISEN_ERR_INVALID, "f32 tensor without a bf16 shadow used in Bf16Mixed mode");
    return t.shadow;
  }
  return t.data;
}

const float* Graph::rope_table(int64_t S, int64_t hd) {
  const int64_t key = S * 100000 + hd;
  auto it = rope_tables_.find(key);
  if (it != rope_tables_.end()) return it->second;
  float* tab = nullptr;
  cuck(cudaMalloc(&tab, (size_t)S * (hd / 2) * 8), "cudaMalloc(rope table)");
  ck(eisen_rope_table(stream, tab, S, hd, 10000.0f), "rope_table");
  rope_tables_[key] = tab;
  return tab;
}

// ------------------------------------------------------------------------------------- streaming
// src/graph/memory.rs:64-125: the residency plan.  Sixteen bytes per element (f32 weight, gradient
// and two AdamW moments) for everything that stays on the device, the largest streamed tensor's
// f32 size as transfer headroom.
StreamingReport Graph::plan_streaming_layout(size_t budget, size_t reserve, const std::vector<int64_t>& pinned) const {
  if (num_params <= 0) invalid("plan_streaming: call mark_params() first");
  auto sat_sub = [](size_t a, size_t b) { return a > b ? a - b : (size_t)0; };
  auto is_param_tensor = [&](int64_t id) { return tensors[(size_t)id].dtype != DT_I32; };
  std::vector<char> is_pinned((size_t)num_params, 0);
  size_t pinned_vram = 0;
  for (int64_t pid : pinned) {
    if (pid < 0 || pid >= num_params || !is_param_tensor(pid)) invalid("plan_streaming: pinned id is not a parameter");
    is_pinned[(size_t)pid] = 1;
    pinned_vram += (size_t)tensors[(size_t)pid].numel * 16;
  }
  const size_t budget_after_fixed = sat_sub(sat_sub(budget, reserve), pinned_vram);
  StreamingReport rep;
  std::vector<int64_t> resident;
  size_t used = 0;
  for (int64_t pid = 0; pid < num_params; ++pid) {
    if (is_pinned[(size_t)pid] || !is_param_tensor(pid)) continue;
    const size_t cost = (size_t)tensors[(size_t)pid].numel * 16;
    if (used + cost <= budget_after_fixed) { used += cost; resident.push_back(pid); }
    else rep.streamed_param_ids.push_back(pid);
  }
  size_t max_stream_bytes = 0;
  for (int64_t pid : rep.streamed_param_ids) max_stream_bytes = std::max(max_stream_bytes, (size_t)tensors[(size_t)pid].numel * 4);
  // make room for one streamed tensor: the largest resident tensor goes first (of equals the last)
  while (max_stream_bytes > sat_sub(budget_after_fixed, used) && !resident.empty()) {
    size_t best = 0;
    for (size_t i = 1; i < resident.size(); ++i)
      if (tensors[(size_t)resident[i]].numel >= tensors[(size_t)resident[best]].numel) best = i;
    const int64_t pid = resident[best];
    resident.erase(resident.begin() + (long)best);
    used -= (size_t)tensors[(size_t)pid].numel * 16;
    rep.streamed_param_ids.push_back(pid);
  }
  for (int64_t pid : rep.streamed_param_ids) rep.streamed_bytes += tensors[(size_t)pid].numel * 4;
  rep.resident_param_ids = pinned;
  rep.resident_param_ids.insert(rep.resident_param_ids.end(), resident.begin(), resident.end());
  for (int64_t pid : rep.resident_param_ids) rep.resident_bytes += tensors[(size_t)pid].numel * 16;
  rep.streaming_headroom_bytes = (int64_t)max_stream_bytes;
  rep.resident_headroom_bytes = 0;  // the reference reports the bytes in use before planning, which is 0
  return rep;
}

StreamingReport Graph::plan_streaming(size_t budget, size_t reserve, const std::vector<int64_t>& pinned) {
  StreamingReport rep = plan_streaming_layout(budget, reserve, pinned);
  cuck(cudaStreamSynchronize(stream), "sync");
  for (int64_t pid : rep.streamed_param_ids) move_param_to_host(pid);
  for (int64_t pid : rep.resident_param_ids) move_param_to_device(pid);
  vram_budget_bytes = budget;
  activation_reserve_bytes = reserve;
  invalidate_staged_weights();
  return rep;
}

// src/graph/memory.rs:323-373 (demote_tensor_to_cpu) for a parameter: data, bf16 copy and gradient
// move to page-locked host memory.  A tensor inside the flat arena keeps its arena range unused.
void Graph::move_param_to_host(int64_t id) {
  HTensor& t = tensors.at(id);
  if (t.host_homed) return;
  if (!t.is_param || t.dtype != 0) invalid("move_param_to_host: not an f32 parameter");
  const size_t n = (size_t)std::max<int64_t>(t.numel, 1);
  void* hd = host_alloc(n * 4);
  void* hg = host_alloc(n * 4);
  void* hs = t.shadow ? host_alloc(n * 2) : nullptr;
  cuck(cudaMemcpy(hd, t.data, n * 4, cudaMemcpyDefault), "D2H(param)");
  cuck(cudaMemcpy(hg, t.grad, n * 4, cudaMemcpyDefault), "D2H(param grad)");
  if (hs) cuck(cudaMemcpy(hs, t.shadow, n * 2, cudaMemcpyDefault), "D2H(param shadow)");
  if (t.owns_data) {
    cudaFree(t.data);
    if (t.shadow) cudaFree(t.shadow);
    device_bytes_allocated -= round256(n * 4) + (t.shadow ? round256(n * 2) : 0);
  }
  if (t.owns_grad) { cudaFree(t.grad); device_bytes_allocated -= round256(n * 4); }
  t.data = hd; t.grad = hg; t.shadow = hs;
  t.owns_data = t.owns_grad = false;
  t.host_homed = true;
}

// src/graph/memory.rs:268-321 (ensure_on_gpu)
void Graph::move_param_to_device(int64_t id) {
  HTensor& t = tensors.at(id);
  if (!t.host_homed) return;
  const size_t n = (size_t)std::max<int64_t>(t.numel, 1);
  void *dd = nullptr, *dg = nullptr, *ds = nullptr;
  cuck(cudaMalloc(&dd, round256(n * 4)), "cudaMalloc(param)");
  cuck(cudaMalloc(&dg, round256(n * 4)), "cudaMalloc(param grad)");
  if (t.shadow) cuck(cudaMalloc(&ds, round256(n * 2)), "cudaMalloc(param shadow)");
  cuck(cudaMemcpy(dd, t.data, n * 4, cudaMemcpyDefault), "H2D(param)");
  cuck(cudaMemcpy(dg, t.grad, n * 4, cudaMemcpyDefault), "H2D(param grad)");
  if (ds) cuck(cudaMemcpy(ds, t.shadow, n * 2, cudaMemcpyDefault), "H2D(param shadow)");
  cudaFreeHost(t.data);
  cudaFreeHost(t.grad);
  if (t.shadow) cudaFreeHost(t.shadow);
  t.data = dd; t.grad = dg; t.shadow = ds;
  t.owns_data = t.owns_grad = true;
  t.host_homed = false;
  device_bytes_allocated += 2 * round256(n * 4) + (ds ? round256(n * 2) : 0);
}

// Staging ring for host-homed GEMM operands.  The reference uploads a streamed weight with a
// blocking copy inside every matmul, forward and backward (src/graph/ops/linear.rs:804-807,
// 893-897); here the copy runs on its own stream into one of a ring of device buffers, early
// when prefetch_weight is called ahead of use, and the compute stream only waits on its event.
constexpr size_t kStageSlots = 16;

void Graph::ensure_stage(size_t bytes) {
  if (!copy_stream_) {
    cuck(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking), "cudaStreamCreate(copy)");
    cuck(cudaEventCreateWithFlags(&compute_mark_, cudaEventDisableTiming), "cudaEventCreate");
  }
  if (bytes <= stage_slot_bytes_ && !stage_.empty()) return;
  // (re)build the ring with slots large enough for this operand
  cuck(cudaStreamSynchronize(stream), "sync");
  cuck(cudaStreamSynchronize(copy_stream_), "sync");
  for (StageSlot& sl : stage_) {
    if (sl.buf) { cudaFree(sl.buf); device_bytes_allocated -= stage_slot_bytes_; }
    sl.buf = nullptr;
    sl.id = -1;
  }
  stage_.resize(kStageSlots);
  stage_slot_bytes_ = round256(bytes);
  for (StageSlot& sl : stage_) {
    cuck(cudaMalloc(&sl.buf, stage_slot_bytes_), "cudaMalloc(weight staging)");
    device_bytes_allocated += stage_slot_bytes_;
    if (!sl.ready) cuck(cudaEventCreateWithFlags(&sl.ready, cudaEventDisableTiming), "cudaEventCreate");
  }
}

Graph::StageSlot* Graph::stage_weight(int64_t id) {
  const HTensor& t = tensors.at(id);
  const bool bf16 = precision == Precision::Bf16Mixed;
  const void* src = bf16 ? t.shadow : t.data;
  if (!src) invalid("weight_operand: host-homed parameter without data");
  const size_t bytes = (size_t)t.numel * (bf16 ? 2 : 4);
  ensure_stage(bytes);
  for (StageSlot& sl : stage_)
    if (sl.id == id && sl.generation == weight_generation_) return &sl;
  StageSlot& sl = stage_[stage_next_];
  stage_next_ = (stage_next_ + 1) % stage_.size();
  // whatever the compute stream has queued so far may still read this slot
  cuck(cudaEventRecord(compute_mark_, stream), "cudaEventRecord");
  cuck(cudaStreamWaitEvent(copy_stream_, compute_mark_, 0), "cudaStreamWaitEvent");
  cuck(cudaMemcpyAsync(sl.buf, src, bytes, cudaMemcpyDefault, copy_stream_), "H2D(weight staging)");
  cuck(cudaEventRecord(sl.ready, copy_stream_), "cudaEventRecord");
  sl.id = id;
  sl.generation = weight_generation_;
  return &sl;
}

void Graph::prefetch_weight(int64_t id) {
  if (tensors.at(id).host_homed) stage_weight(id);
}

const void* Graph::weight_operand(int64_t id) {
  const HTensor& t = tensors.at(id);
  if (!t.host_homed) return operand(t);
  StageSlot* sl = stage_weight(id);
  cuck(cudaStreamWaitEvent(stream, sl->ready, 0), "cudaStreamWaitEvent");
  return sl->buf;
}

void Graph::prof_begin(int cls, double flops) {
  if (!prof_on) return;
  ProfRec r;
  auto get = [this]() {
    cudaEvent_t e;
    if (!prof_free.empty()) { e = prof_free.back(); prof_free.pop_back(); }
    else cuck(cudaEventCreate(&e), "cudaEventCreate");
    return e;
  };
  r.a = get();
  r.b = get();
  r.flops = flops;
  r.cls = cls;
  cuck(cudaEventRecord(r.a, stream), "cudaEventRecord");
  prof_recs.push_back(r);
}
void Graph::prof_end() {
  if (!prof_on || prof_recs.empty()) return;
  cuck(cudaEventRecord(prof_recs.back().b, stream), "cudaEventRecord");
}
void Graph::prof_read(double* out9) {
  for (int i = 0; i < 9; ++i) out9[i] = 0.0;
  cuck(cudaStreamSynchronize(stream), "sync");
  for (ProfRec& r : prof_recs) {
    float ms = 0.0f;
    cuck(cudaEventElapsedTime(&ms, r.a, r.b), "cudaEventElapsedTime");
    out9[r.cls * 3 + 0] += ms;
    out9[r.cls * 3 + 1] += r.flops;
    out9[r.cls * 3 + 2] += 1.0;
    prof_free.push_back(r.a);
    prof_free.push_back(r.b);
  }
  prof_recs.clear();
}

// helper: true if the output carries a gradient worth propagating
#define OUT_GRAD_OR_RETURN(o)                         \
  HTensor& to = tensors[o];                           \
  if (!to.grad || !to.grad_init) return;

// ------------------------------------------------------------------------------------- elementwise
// src/graph/ops/elementwise.rs:7-186 — b may broadcast over leading dims (bias, [1,S,S] mask)
int64_t Graph::add(int64_t a, int64_t b) {
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  if (tb.numel == 0 || ta.numel % tb.numel) invalid("add: rhs must match or broadcast over leading dims");
  const int dt = act_dtype();
  const int64_t n = ta.numel, bn = tb.numel;
  int64_t o = alloc_pooled(ta.shape);
  if (!skip_forward)
    ck(eisen_add(stream, operand(tensors[a]), operand(tensors[b]), tensors[o].data, n, bn, dt), "add");
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, n, bn]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      if (!ga.constant) {
        ensure_grad(a);
        ck(eisen_accumulate(stream, ga.grad, ga.grad_dtype, to.grad, to.grad_dtype, n, ga.grad_init), "add.bwd(a)");
        ga.grad_init = true;
      }
      HTensor& gb = tensors[b];
      if (!gb.constant) {
        ensure_grad(b);
        if (bn == n) {
          ck(eisen_accumulate(stream, gb.grad, gb.grad_dtype, to.grad, to.grad_dtype, n, gb.grad_init), "add.bwd(b)");
        } else {
          if (gb.grad_dtype != 0) invalid("add: broadcast operand needs an f32 gradient");
          ck(eisen_reduce_leading(stream, to.grad, to.grad_dtype, static_cast<float*>(gb.grad), n, bn, gb.grad_init), "add.bwd(b)");
        }
        gb.grad_init = true;
      }
    }});
  }
  return o;
}

// src/graph/ops/elementwise.rs:188-334 (no broadcast)
int64_t Graph::mul(int64_t a, int64_t b) {
  const HTensor& ta = tensors.at(a);
  if (ta.numel != tensors.at(b).numel) invalid("mul: shapes differ");
  const int dt = act_dtype();
  const int64_t n = ta.numel;
  int64_t o = alloc_pooled(ta.shape);
  ck(eisen_mul_fwd(stream, operand(tensors[a]), operand(tensors[b]), tensors[o].data, n, dt), "mul");
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, n, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      void* da = nullptr;
      void* db = nullptr;
      if (!ga.constant) { ensure_grad(a); da = ga.grad; }
      if (!gb.constant) { ensure_grad(b); db = gb.grad; }
      if ((da && ga.grad_dtype != dt) || (db && gb.grad_dtype != dt)) invalid("mul: gradient dtype differs from the activation dtype");
      ck(eisen_mul_bwd(stream, operand(ga), operand(gb), to.grad, da, db, n, dt, ga.grad_init, gb.grad_init), "mul.bwd");
      if (da) ga.grad_init = true;
      if (db) gb.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/elementwise.rs:337-467
int64_t Graph::silu(int64_t a) {
  const int dt = act_dtype();
  const int64_t n = tensors.at(a).numel;
  int64_t o = alloc_pooled(tensors[a].shape);
  ck(eisen_silu_fwd(stream, operand(tensors[a]), tensors[o].data, n, dt), "silu");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, n, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      ck(eisen_silu_bwd(stream, operand(ga), to.grad, ga.grad, n, dt, ga.grad_init), "silu.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

// silu(gate) * up in one pass each way (src/nn/transformer.rs:41-44 uses silu + mul)
int64_t Graph::swiglu(int64_t gate, int64_t up) {
  const int dt = act_dtype();
  const int64_t n = tensors.at(gate).numel;
  if (tensors.at(up).numel != n) invalid("swiglu: shapes differ");
  int64_t o = alloc_pooled(tensors[gate].shape);
  if (!skip_forward)
    ck(eisen_swiglu_fwd(stream, operand(tensors[gate]), operand(tensors[up]), tensors[o].data, n, dt), "swiglu");
  if (!no_grad) {
    tape.push_back({{gate, up}, o, [this, gate, up, o, n, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& gg = tensors[gate];
      HTensor& gu = tensors[up];
      ensure_grad(gate);
      ensure_grad(up);
      if (gg.grad_init != gu.grad_init) invalid("swiglu: gate and up gradients must both be fresh or both initialised");
      ck(eisen_swiglu_bwd(stream, operand(gg), operand(gu), to.grad, gg.grad, gu.grad, n, dt, gg.grad_init), "swiglu.bwd");
      gg.grad_init = gu.grad_init = true;
    }});
  }
  return o;
}

// ------------------------------------------------------------------------------------- contractions
namespace {
// C[m,n] (op)= A(m,k) B(n,k) with per-operand major, dispatched on the graph precision.
// a_mn / b_mn as in eisen_gemm_bf16; strides are the row lengths of the stored matrices.
void gemm(Graph& g, bool a_mn, bool b_mn, int64_t M, int64_t N, int64_t K, const void* A, const void* B, void* C,
          int c_dtype, bool accumulate) {
  if (g.precision == Precision::Fp32) {
    const int64_t a_ms = a_mn ? 1 : K, a_ks = a_mn ? M : 1;
    const int64_t b_ns = b_mn ? 1 : K, b_ks = b_mn ? N : 1;
    ck(eisen_gemm_f32_strided(g.stream, (const float*)A, (const float*)B, (float*)C, 1, M, N, K, 0, a_ms, a_ks, 0,
                              b_ks, b_ns, 0, N, accumulate),
       "gemm_f32");
    return;
  }
  const int64_t lda = a_mn ? M : K, ldb = b_mn ? N : K;
  int mode;
  if (c_dtype == 1) mode = accumulate ? 1 : 0;
  else mode = accumulate ? 4 : 2;  // f32 accumulation goes through red.global.add with automatic split-K
  g.prof_begin(0, 2.0 * (double)M * (double)N * (double)K);
  ck(eisen_gemm_bf16(g.stream, a_mn, b_mn, M, N, K, A, lda, B, ldb, C, N, mode, mode == 4 ? 0 : 1, 1.0f, g.status_dev),
     "gemm_bf16");
  g.prof_end();
}

// Weight gradient dW[M,N] (+)= A(m,k) B(n,k) into parameter (or activation) `w`.  A host-homed
// parameter keeps its gradient in host memory: the product goes to a pooled device buffer and is
// then added to the host gradient by a plain element kernel (the reference downloads the product
// and adds it on the CPU, src/graph/ops/linear.rs:937-947).
void dw_gemm(Graph& g, bool a_mn, bool b_mn, int64_t M, int64_t N, int64_t K, const void* A, const void* B, int64_t w) {
  HTensor& gw = g.tensors[w];
  if (!gw.host_homed) {
    gemm(g, a_mn, b_mn, M, N, K, A, B, gw.grad, gw.grad_dtype, gw.grad_init);
  } else {
    const size_t bytes = (size_t)M * N * 4;
    void* tmp = g.pool_get(bytes);
    struct Release { Graph& g; void* p; size_t b; ~Release() { g.pool_put(p, b); } } release{g, tmp, bytes};
    gemm(g, a_mn, b_mn, M, N, K, A, B, tmp, 0, false);
    ck(eisen_accumulate(g.stream, gw.grad, 0, tmp, 0, M * N, gw.grad_init), "dW(host-homed)");
  }
  gw.grad_init = true;
}
}  // namespace

// src/graph/ops/linear.rs:35-299 (f32) and 526-770 (bf16 operands): C[m,n] = A[m,k] B[k,n]
int64_t Graph::matmul(int64_t a, int64_t b) {
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  if (ta.shape.size() < 2) invalid("matmul: lhs must have rank >= 2");
  if (tb.shape.size() != 2) invalid("matmul: rhs must have rank 2 [k, n]");
  const int64_t k = ta.shape.back(), m = ta.numel / k, n = tb.shape[1];
  if (tb.shape[0] != k) invalid("matmul: lhs last dim must equal rhs first dim");
  int64_t o = alloc_pooled({m, n});
  if (!skip_forward)
    gemm(*this, false, true, m, n, k, operand(tensors[a]), weight_operand(b), tensors[o].data, act_dtype(), false);
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, m, n, k]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      if (!ga.constant) {  // dA[m,k] (+)= dC[m,n] B[k,n]^T
        ensure_grad(a);
        gemm(*this, false, false, m, k, n, to.grad, weight_operand(b), ga.grad, ga.grad_dtype, ga.grad_init);
        ga.grad_init = true;
      }
      if (!gb.constant) {  // dB[k,n] (+)= A[m,k]^T dC[m,n]
        ensure_grad(b);
        dw_gemm(*this, true, true, k, n, m, operand(ga), to.grad, b);
      }
    }});
  }
  return o;
}

// rope(x W): a `Linear` followed by RoPE (src/nn/attention.rs:320-333) with the rotation in the GEMM
// epilogue.  Backward: the incoming gradient is rotated back in place, then the two products of
// matmul's backward.  Shapes the fused kernel does not take (and Fp32 graphs) run matmul + rope.
int64_t Graph::matmul_rope(int64_t a, int64_t b, int64_t head_dim) {
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  if (ta.shape.size() != 3) invalid("matmul_rope: lhs must be [batch, seq, k]");
  if (tb.shape.size() != 2) invalid("matmul_rope: rhs must have rank 2 [k, n]");
  const int64_t B = ta.shape[0], S = ta.shape[1], k = ta.shape[2], m = B * S, n = tb.shape[1];
  if (tb.shape[0] != k) invalid("matmul_rope: lhs last dim must equal rhs first dim");
  const bool fusable = precision == Precision::Bf16Mixed && m % 256 == 0 && n % 256 == 0 && k % 8 == 0 &&
                       head_dim % 8 == 0 && n % head_dim == 0;
  if (!fusable) {
    int64_t o = matmul(a, b);
    reinterpret_shape(o, {B, S, n});
    return rope(o, head_dim);
  }
  const float* tab = rope_table(S, head_dim);
  const int dt = act_dtype();
  int64_t o = alloc_pooled({B, S, n});
  if (!skip_forward) {
    prof_begin(0, 2.0 * (double)m * (double)n * (double)k);
    ck(eisen_gemm_bf16_rope(stream, m, n, k, operand(tensors[a]), k, weight_operand(b), n, tensors[o].data, n, tab, S,
                            head_dim, status_dev),
       "matmul_rope");
    prof_end();
  }
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, B, S, m, n, k, head_dim, dt, tab]() {
      OUT_GRAD_OR_RETURN(o);
      // the rotated gradient goes to a pooled temporary: the output's own gradient stays as the
      // consumer wrote it, so a tape that is walked again (the reference keeps its nodes) sees it unchanged
      const size_t rot_bytes = (size_t)m * n * dsize(dt);
      void* rot = pool_get(rot_bytes);
      struct Release { Graph& g; void* p; size_t b; ~Release() { g.pool_put(p, b); } } release{*this, rot, rot_bytes};
      ck(eisen_rope(stream, to.grad, rot, tab, B, S, n, head_dim, dt, 1, 0), "matmul_rope.bwd(rope)");
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      if (!ga.constant) {
        ensure_grad(a);
        gemm(*this, false, false, m, k, n, rot, weight_operand(b), ga.grad, ga.grad_dtype, ga.grad_init);
        ga.grad_init = true;
      }
      if (!gb.constant) {
        ensure_grad(b);
        dw_gemm(*this, true, true, k, n, m, operand(ga), rot, b);
      }
    }});
  }
  return o;
}

// The three projections of GroupedQueryAttention::forward_with_mask (src/nn/attention.rs:316-333:
// q_proj, k_proj, v_proj on one input, RoPE on q and k) as one tape entry.  Forward: one launch
// whose n-tiles are spread over the three weights (RoPE in the epilogue of the q and k tiles).
// Backward: dX = dQ' Wq^T + dK' Wk^T + dV Wv^T in one pass over the three operand pairs (dQ', dK' =
// the gradients rotated back), and the three dW = X^T dY in one launch.  Shapes the fused kernels do
// not take, Fp32 graphs and host-homed weights run matmul_rope, matmul_rope, matmul.
// The q and k it returns are meant for Graph::attention alone: that op's backward hands their
// gradients over rotated back already (HTensor::unrope_hd / grad_unrotated), which a second consumer
// adding a gradient in the rotated form would not match.
void Graph::qkv_proj_rope(int64_t x, int64_t wq, int64_t wk, int64_t wv, int64_t head_dim, int64_t out3[3]) {
  const HTensor& tx = tensors.at(x);
  const int64_t ws[3] = {wq, wk, wv};
  bool fusable = precision == Precision::Bf16Mixed && tx.shape.size() == 3 && head_dim % 8 == 0 && head_dim >= 8;
  int64_t B = 0, S = 0, k = 0, m = 0;
  long long ns[3] = {0, 0, 0};
  if (fusable) {
    B = tx.shape[0]; S = tx.shape[1]; k = tx.shape[2]; m = B * S;
    fusable = m % 256 == 0 && k % 8 == 0;
    for (int i = 0; i < 3 && fusable; ++i) {
      const HTensor& tw = tensors.at(ws[i]);
      fusable = tw.shape.size() == 2 && tw.shape[0] == k && tw.shape[1] % 256 == 0 && tw.shape[1] % head_dim == 0 &&
                !tw.host_homed && !tw.constant && tw.grad_dtype == 0;
      ns[i] = fusable ? tw.shape[1] : 0;
    }
    fusable = fusable && !tx.constant;
  }
  if (!fusable) {
    out3[0] = matmul_rope(x, wq, head_dim);
    out3[1] = matmul_rope(x, wk, head_dim);
    out3[2] = matmul(x, wv);
    if (tensors.at(x).shape.size() == 3)
      reinterpret_shape(out3[2], {tensors[x].shape[0], tensors[x].shape[1], tensors.at(wv).shape[1]});
    return;
  }
  const float* tab = rope_table(S, head_dim);
  const int dt = act_dtype();
  // With Graph::center_values the value projection is written in f32: Graph::attention then subtracts the
  // values' mean before rounding them to bf16, which keeps their token-specific part to bf16 precision.
  const bool v_f32 = center_values;
  for (int i = 0; i < 2; ++i) out3[i] = alloc_pooled({B, S, ns[i]});
  out3[2] = v_f32 ? alloc_pooled_dtype({B, S, ns[2]}, 0) : alloc_pooled({B, S, ns[2]});
  const int64_t oq = out3[0], ok = out3[1], ov = out3[2];
  tensors[ov].grad_dtype = dt;  // the attention backward writes dv in the activation type
  tensors[oq].unrope_hd = tensors[ok].unrope_hd = head_dim;
  if (!skip_forward) {
    const void* bs[3] = {weight_operand(wq), weight_operand(wk), weight_operand(wv)};
    void* cs[3] = {tensors[oq].data, tensors[ok].data, tensors[ov].data};
    const int modes[3] = {5, 5, v_f32 ? 2 : 0};
    prof_begin(0, 2.0 * (double)m * (double)(ns[0] + ns[1] + ns[2]) * (double)k);
    ck(eisen_gemm_bf16_multi_n(stream, 0, 1, m, k, operand(tensors[x]), k, 3, bs, ns, ns, cs, ns, modes, 1, 1.0f, tab, S,
                               head_dim, status_dev),
       "qkv_proj_rope");
    prof_end();
  }
  if (no_grad) return;
  const long long n0 = ns[0], n1 = ns[1], n2 = ns[2];
  tape.push_back({{x, wq, wk, wv}, ov, [this, x, wq, wk, wv, oq, ok, ov, B, S, m, k, n0, n1, n2, head_dim, dt, tab]() {
    const int64_t outs[3] = {oq, ok, ov}, ws[3] = {wq, wk, wv};
    const long long ns[3] = {n0, n1, n2};
    bool have[3];
    int n_have = 0;
    for (int i = 0; i < 3; ++i) {
      const HTensor& to = tensors[outs[i]];
      have[i] = to.grad && to.grad_init;
      n_have += have[i];
    }
    if (!n_have) return;
    // the gradients of q and k are rotated back into pooled temporaries (the outputs' own gradients
    // stay as their consumer wrote them, so the tape can be walked again)
    struct Temp { Graph& g; void* p; size_t b; ~Temp() { if (p) g.pool_put(p, b); } };
    Temp rq{*this, nullptr, 0}, rk{*this, nullptr, 0};
    const void* dy[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < 2; ++i) {
      if (!have[i]) continue;
      if (tensors[outs[i]].grad_unrotated) {  // the attention backward delivered it rotated back already
        dy[i] = tensors[outs[i]].grad;
        continue;
      }
      Temp& t = i == 0 ? rq : rk;
      t.b = (size_t)m * ns[i] * dsize(dt);
      t.p = pool_get(t.b);
      ck(eisen_rope(stream, tensors[outs[i]].grad, t.p, tab, B, S, ns[i], head_dim, dt, 1, 0), "qkv_proj_rope.bwd(rope)");
      dy[i] = t.p;
    }
    if (have[2]) dy[2] = tensors[ov].grad;
    HTensor& gx = tensors[x];
    ensure_grad(x);
    for (int i = 0; i < 3; ++i) ensure_grad(ws[i]);
    if (n_have == 3 && gx.grad_dtype == 1) {
      // dX (op)= sum_i dY_i W_i^T, one pass over the three operand pairs
      const void* as[3] = {dy[0], dy[1], dy[2]};
      const void* bs[3] = {weight_operand(wq), weight_operand(wk), weight_operand(wv)};
      prof_begin(0, 2.0 * (double)m * (double)(n0 + n1 + n2) * (double)k);
      ck(eisen_gemm_bf16_concat_k(stream, 0, 0, m, k, 3, as, ns, bs, ns, ns, gx.grad, k, gx.grad_init ? 1 : 0, 1, 1.0f,
                                  status_dev),
         "qkv_proj_rope.bwd(dX)");
      prof_end();
      gx.grad_init = true;
      // dW_i (+)= X^T dY_i, one launch over the n-tiles of the three gradients
      bool fresh = false;
      for (int i = 0; i < 3; ++i) fresh = fresh || !tensors[ws[i]].grad_init;
      if (!fresh) {
        void* cs[3] = {tensors[wq].grad, tensors[wk].grad, tensors[wv].grad};
        const int modes[3] = {4, 4, 4};
        prof_begin(0, 2.0 * (double)m * (double)(n0 + n1 + n2) * (double)k);
        ck(eisen_gemm_bf16_multi_n(stream, 1, 1, k, m, operand(gx), k, 3, dy, ns, ns, cs, ns, modes, 0, 1.0f, nullptr, 0, 0,
                                   status_dev),
           "qkv_proj_rope.bwd(dW)");
        prof_end();
        return;
      }
      for (int i = 0; i < 3; ++i) dw_gemm(*this, true, true, k, ns[i], m, operand(gx), dy[i], ws[i]);
      return;
    }
    for (int i = 2; i >= 0; --i) {  // the order in which the separate tape entries would run
      if (!have[i]) continue;
      gemm(*this, false, false, m, k, ns[i], dy[i], weight_operand(ws[i]), gx.grad, gx.grad_dtype, gx.grad_init);
      gx.grad_init = true;
      dw_gemm(*this, true, true, k, ns[i], m, operand(gx), dy[i], ws[i]);
    }
  }});
}

// silu(x Wg) * (x Wu): the gate and up `Linear`s and the SiLU-gated product of
// src/nn/transformer.rs:41-44 in one launch.  The tape gets the same three entries as
// matmul, matmul, swiglu (their forward kernels are skipped), so the backward pass is theirs.
// Shapes the fused kernel does not take (and Fp32 graphs) run the three ops.
int64_t Graph::gate_up_swiglu(int64_t x, int64_t wg, int64_t wu) {
  const HTensor& tx = tensors.at(x);
  const HTensor& tg = tensors.at(wg);
  const HTensor& tu = tensors.at(wu);
  if (tg.shape.size() != 2 || tu.shape != tg.shape) invalid("gate_up_swiglu: weights must be two [k, n] matrices");
  const int64_t k = tx.shape.back(), m = tx.numel / k, n = tg.shape[1];
  if (tg.shape[0] != k) invalid("gate_up_swiglu: lhs last dim must equal the weights' first dim");
  const bool fusable = precision == Precision::Bf16Mixed && m % 256 == 0 && n % 128 == 0 && k % 8 == 0 && !skip_forward;
  if (!fusable) {
    int64_t go = matmul(x, wg);
    int64_t up = matmul(x, wu);
    return swiglu(go, up);
  }
  const double flops = 4.0 * (double)m * (double)n * (double)k;
  if (no_grad) {  // nothing is kept for a backward pass: only the product is written
    int64_t h = alloc_pooled({m, n});
    prof_begin(0, flops);
    ck(eisen_gemm_bf16_swiglu(stream, m, n, k, operand(tensors[x]), k, weight_operand(wg), weight_operand(wu), n,
                              nullptr, nullptr, tensors[h].data, n, status_dev),
       "gate_up_swiglu");
    prof_end();
    return h;
  }
  int64_t go, up, h;
  {
    FlagGuard skip(skip_forward, true);
    go = matmul(x, wg);
    up = matmul(x, wu);
    h = swiglu(go, up);
  }
  prof_begin(0, flops);
  ck(eisen_gemm_bf16_swiglu(stream, m, n, k, operand(tensors[x]), k, weight_operand(wg), weight_operand(wu), n,
                            tensors[go].data, tensors[up].data, tensors[h].data, n, status_dev),
     "gate_up_swiglu");
  prof_end();
  return h;
}

// out[m,n] = r[m,n] + a[m,k] b[k,n]: `Linear` followed by the residual `add` of
// src/nn/transformer.rs:36, 47, with the add folded into the GEMM epilogue (Bf16Mixed only)
int64_t Graph::matmul_add(int64_t a, int64_t b, int64_t r) {
  if (precision != Precision::Bf16Mixed) invalid("matmul_add: fused residual epilogue runs in Bf16Mixed mode");
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  const HTensor& tr = tensors.at(r);
  if (tb.shape.size() != 2) invalid("matmul_add: rhs must have rank 2 [k, n]");
  const int64_t k = ta.shape.back(), m = ta.numel / k, n = tb.shape[1];
  if (tb.shape[0] != k || tr.numel != m * n) invalid("matmul_add: shape mismatch");
  int64_t o = alloc_pooled(tr.shape);
  if (!skip_forward) {
    prof_begin(0, 2.0 * (double)m * (double)n * (double)k);
    ck(eisen_gemm_bf16_residual(stream, 0, 1, m, n, k, operand(tensors[a]), k, weight_operand(b), n, operand(tensors[r]),
                                n, tensors[o].data, n, 1.0f, status_dev),
       "matmul_add");
    prof_end();
  }
  if (!no_grad) {
    tape.push_back({{a, b, r}, o, [this, a, b, r, o, m, n, k]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      HTensor& gr = tensors[r];
      const bool move_to_r = !gr.constant && gr.grad == nullptr && gr.is_pooled && to.is_pooled &&
                             gr.grad_dtype == to.grad_dtype && gr.numel == to.numel;
      if (!gr.constant && !move_to_r) {  // dR (+)= dOut
        ensure_grad(r);
        ck(eisen_accumulate(stream, gr.grad, gr.grad_dtype, to.grad, to.grad_dtype, m * n, gr.grad_init), "matmul_add.bwd(r)");
        gr.grad_init = true;
      }
      struct MoveGrad {  // dR = dOut without a copy: the output's gradient buffer becomes the residual's
        HTensor& from; HTensor& dst; bool on;
        ~MoveGrad() { if (on) { dst.grad = from.grad; dst.grad_init = true; from.grad = nullptr; from.grad_init = false; } }
      } mover{to, gr, move_to_r};
      if (!ga.constant) {
        ensure_grad(a);
        gemm(*this, false, false, m, k, n, to.grad, weight_operand(b), ga.grad, ga.grad_dtype, ga.grad_init);
        ga.grad_init = true;
      }
      if (!gb.constant) {
        ensure_grad(b);
        dw_gemm(*this, true, true, k, n, m, operand(ga), to.grad, b);
      }
    }});
  }
  return o;
}

// src/graph/ops/linear.rs:301-523 (tied LM head): C[m,n] = A[m,k] B[n,k]^T
int64_t Graph::matmul_trans_b(int64_t a, int64_t b) {
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  if (tb.shape.size() != 2) invalid("matmul_trans_b: rhs must have rank 2 [n, k]");
  const int64_t k = ta.shape.back(), m = ta.numel / k, n = tb.shape[0];
  if (tb.shape[1] != k) invalid("matmul_trans_b: inner dims differ");
  int64_t o = alloc_pooled({m, n});
  gemm(*this, false, false, m, n, k, operand(tensors[a]), weight_operand(b), tensors[o].data, act_dtype(), false);
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, m, n, k]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      if (!ga.constant) {  // dA[m,k] (+)= dC[m,n] B[n,k]
        ensure_grad(a);
        gemm(*this, false, true, m, k, n, to.grad, weight_operand(b), ga.grad, ga.grad_dtype, ga.grad_init);
        ga.grad_init = true;
      }
      if (!gb.constant) {  // dB[n,k] (+)= dC[m,n]^T A[m,k]
        ensure_grad(b);
        dw_gemm(*this, true, true, n, k, m, to.grad, operand(ga), b);
      }
    }});
  }
  return o;
}

// src/graph/ops/linear.rs:1198-1512; f32 only (the bf16 path uses the fused attention op)
int64_t Graph::bmm(int64_t a, int64_t b, bool trans_b) {
  if (precision != Precision::Fp32) invalid("bmm: only the Fp32 graph materialises attention scores; use attention()");
  const HTensor& ta = tensors.at(a);
  const HTensor& tb = tensors.at(b);
  if (ta.shape.size() != 3 || tb.shape.size() != 3) invalid("bmm: operands must be [batch, m, k]");
  const int64_t batch = ta.shape[0], m = ta.shape[1], k = ta.shape[2];
  const int64_t n = trans_b ? tb.shape[1] : tb.shape[2];
  if (tb.shape[0] != batch || (trans_b ? tb.shape[2] : tb.shape[1]) != k) invalid("bmm: shape mismatch");
  int64_t o = alloc_pooled({batch, m, n});
  const int64_t b_ks = trans_b ? 1 : n, b_ns = trans_b ? k : 1;
  ck(eisen_gemm_f32_strided(stream, (const float*)tensors[a].data, (const float*)tensors[b].data, (float*)tensors[o].data,
                            batch, m, n, k, m * k, k, 1, k * n, b_ks, b_ns, m * n, n, 0),
     "bmm");
  if (!no_grad) {
    tape.push_back({{a, b}, o, [this, a, b, o, batch, m, n, k, trans_b, b_ks, b_ns]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      HTensor& gb = tensors[b];
      const float* dC = (const float*)to.grad;
      if (!ga.constant) {  // dA[b,m,k] (+)= sum_n dC[b,m,n] B(b,k,n)
        ensure_grad(a);
        ck(eisen_gemm_f32_strided(stream, dC, (const float*)gb.data, (float*)ga.grad, batch, m, k, n, m * n, n, 1, k * n,
                                  b_ns, b_ks, m * k, k, ga.grad_init),
           "bmm.bwd(a)");
        ga.grad_init = true;
      }
      if (!gb.constant) {
        ensure_grad(b);
        if (trans_b) {  // dB[b,n,k] (+)= sum_m dC[b,m,n] A[b,m,k]
          ck(eisen_gemm_f32_strided(stream, dC, (const float*)ga.data, (float*)gb.grad, batch, n, k, m, m * n, 1, n, m * k,
                                    k, 1, n * k, k, gb.grad_init),
             "bmm.bwd(b)");
        } else {        // dB[b,k,n] (+)= sum_m A[b,m,k] dC[b,m,n]
          ck(eisen_gemm_f32_strided(stream, (const float*)ga.data, dC, (float*)gb.grad, batch, k, n, m, m * k, 1, k, m * n,
                                    n, 1, k * n, n, gb.grad_init),
             "bmm.bwd(b)");
        }
        gb.grad_init = true;
      }
    }});
  }
  return o;
}

// ------------------------------------------------------------------------------------- row ops
// src/graph/ops/reduction.rs:397-526
int64_t Graph::softmax(int64_t a) {
  const HTensor& ta = tensors.at(a);
  const int dt = act_dtype();
  const int64_t n = ta.shape.back(), rows = ta.numel / n;
  int64_t o = alloc_pooled(ta.shape);
  ck(eisen_softmax_fwd(stream, operand(tensors[a]), tensors[o].data, rows, n, dt), "softmax");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, rows, n, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      ck(eisen_softmax_bwd(stream, to.data, to.grad, ga.grad, rows, n, dt, ga.grad_init), "softmax.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

int64_t Graph::ce_impl(int64_t logits, const int64_t* targets, int64_t n, bool masked, float normalizer) {
  const HTensor& tl = tensors.at(logits);
  if (tl.shape.size() != 2 || tl.shape[0] != n) invalid("cross_entropy: logits must be [rows, classes] with one target per row");
  const int64_t rows = tl.shape[0], vocab = tl.shape[1];
  // targets -> device int32; IGNORE_INDEX (usize::MAX in the reference, any negative value here) -> -1
  std::vector<int32_t> h((size_t)rows);
  for (int64_t i = 0; i < rows; ++i) {
    if (targets[i] < 0) h[i] = -1;
    else if (targets[i] >= vocab) invalid("cross_entropy: target out of range");
    else h[i] = (int32_t)targets[i];
  }
  (void)masked;
  int64_t tid = alloc_ids({rows}, h.data(), false);
  return ce_device(logits, tid, normalizer);
}

int64_t Graph::ce_device(int64_t logits, int64_t tid, float normalizer) {
  const HTensor& tl = tensors.at(logits);
  if (tl.shape.size() != 2) invalid("cross_entropy: logits must be [rows, classes]");
  const int64_t rows = tl.shape[0], vocab = tl.shape[1];
  if (tensors.at(tid).dtype != DT_I32 || tensors[tid].numel != rows) invalid("cross_entropy: one int32 target per row expected");
  const int dt = act_dtype();
  int64_t lse = alloc_pooled_dtype({rows}, 0);
  int64_t row_loss = alloc_pooled_dtype({rows}, 0);
  int64_t o = alloc_pooled_dtype({}, 0);
  tensors[lse].constant = tensors[row_loss].constant = true;
  ck(eisen_ce_fwd(stream, operand(tensors[logits]), (const int*)tensors[tid].data, (float*)tensors[o].data,
                  (float*)tensors[row_loss].data, (float*)tensors[lse].data, rows, vocab, -1, normalizer, dt,
                  bad_id_dev + 1),
     "cross_entropy");
  if (!no_grad) {
    tape.push_back({{logits}, o, [this, logits, tid, lse, o, rows, vocab, normalizer, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& gl = tensors[logits];
      ensure_grad(logits);
      ck(eisen_ce_bwd(stream, operand(gl), (const int*)tensors[tid].data, (const float*)tensors[lse].data, gl.grad,
                      (const float*)to.grad, rows, vocab, -1, normalizer, dt, gl.grad_init),
         "cross_entropy.bwd");
      gl.grad_init = true;
    }});
  }
  return o;
}

// src/nn/transformer.rs:189-195 (`Linear` head, or `matmul_trans_b` with the tied table) followed by
// src/graph/ops/reduction.rs:529-944 (cross_entropy[_masked]) and their backward kernels, as one op
// that never holds more than a [chunk_rows, vocab] slab of logits.
int64_t Graph::lm_head_cross_entropy(int64_t h, int64_t w, int64_t tid, float normalizer, bool trans_b,
                                     int64_t chunk_rows) {
  const HTensor& th = tensors.at(h);
  const HTensor& tw = tensors.at(w);
  if (tw.shape.size() != 2) invalid("lm_head_cross_entropy: the head weight must have rank 2");
  const int64_t k = th.shape.back(), rows = th.numel / k;
  const int64_t vocab = trans_b ? tw.shape[0] : tw.shape[1];
  if ((trans_b ? tw.shape[1] : tw.shape[0]) != k) invalid("lm_head_cross_entropy: inner dims differ");
  if (tensors.at(tid).dtype != DT_I32 || tensors[tid].numel != rows) invalid("lm_head_cross_entropy: one int32 target per row expected");
  if (chunk_rows <= 0 || chunk_rows > rows) chunk_rows = rows;
  const int dt = act_dtype();
  const bool grads = !no_grad;
  int64_t row_loss = alloc_pooled_dtype({rows}, 0);
  int64_t o = alloc_pooled_dtype({}, 0);
  tensors[row_loss].constant = true;
  if (grads) {
    ensure_grad(h);
    if (!tensors[w].constant) ensure_grad(w);
    if (tensors[h].grad_dtype != dt) invalid("lm_head_cross_entropy: the hidden-state gradient must have the activation dtype");
  }
  const size_t slab_bytes = (size_t)chunk_rows * vocab * dsize(dt);
  void* slab = pool_get(slab_bytes);
  struct Release { Graph& g; void* p; size_t b; ~Release() { g.pool_put(p, b); } } release{*this, slab, slab_bytes};
  const int* targets = (const int*)tensors[tid].data;
  float* rl = (float*)tensors[row_loss].data;
  for (int64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
    const int64_t m = std::min(chunk_rows, rows - r0);
    const char* hrows = (const char*)operand(tensors[h]) + (size_t)r0 * k * dsize(dt);
    // logits of these rows: [m, vocab] = H[m, k] W[k, vocab]  (tied: W^T with W [vocab, k])
    gemm(*this, false, !trans_b, m, vocab, k, hrows, weight_operand(w), slab, dt, false);
    if (!grads) {
      ck(eisen_ce_fwd(stream, slab, targets + r0, nullptr, rl + r0, nullptr, m, vocab, -1, normalizer, dt, bad_id_dev + 1),
         "lm_head_cross_entropy(loss)");
      continue;
    }
    ck(eisen_ce_fused(stream, slab, targets + r0, nullptr, rl + r0, nullptr, m, vocab, -1, normalizer, 1.0f, dt, bad_id_dev + 1),
       "lm_head_cross_entropy(ce)");
    HTensor& gh = tensors[h];
    HTensor& gw = tensors[w];
    // dH rows (op)= dlogits W^T
    char* dh = (char*)gh.grad + (size_t)r0 * k * dsize(gh.grad_dtype);
    gemm(*this, false, trans_b, m, k, vocab, slab, weight_operand(w), dh, gh.grad_dtype, gh.grad_init);
    if (!gw.constant) {
      // dW (op)= H^T dlogits  (tied: dW[vocab, k] (op)= dlogits^T H)
      if (!trans_b) dw_gemm(*this, true, true, k, vocab, m, hrows, slab, w);
      else dw_gemm(*this, true, true, vocab, k, m, slab, hrows, w);
    }
  }
  if (grads) tensors[h].grad_init = true;
  ck(eisen_ce_loss_reduce(stream, rl, (float*)tensors[o].data, rows), "lm_head_cross_entropy(reduce)");
  if (grads) {
    tape.push_back({{h, w}, o, [this, o]() {
      OUT_GRAD_OR_RETURN(o);
      if (!to.grad_is_ones)
        invalid("lm_head_cross_entropy: its gradients are formed in the forward with a loss gradient of 1; "
                "the loss must be the tensor backward() starts from");
    }});
  }
  return o;
}

// src/graph/ops/reduction.rs:529-719: mean over rows of -ln(p_target + 1e-8)
int64_t Graph::cross_entropy(int64_t logits, const int64_t* targets, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    if (targets[i] < 0) invalid("cross_entropy: negative target (use cross_entropy_masked for ignored rows)");
  return ce_impl(logits, targets, n, false, 1.0f / (float)n);
}

// src/graph/ops/reduction.rs:724-737: plain CE when nothing is masked, constant 0 when all is
int64_t Graph::cross_entropy_masked(int64_t logits, const int64_t* targets, int64_t n) {
  int64_t valid = 0;
  for (int64_t i = 0; i < n; ++i) valid += (targets[i] >= 0);
  if (valid == n) return cross_entropy(logits, targets, n);
  if (valid == 0) {
    int64_t o = alloc_pooled_dtype({}, 0);
    cuck(cudaMemsetAsync(tensors[o].data, 0, 4, stream), "memset");
    return o;
  }
  return ce_impl(logits, targets, n, true, 1.0f / (float)valid);
}

// src/graph/ops/normalization.rs:8-183
int64_t Graph::rms_norm(int64_t x, int64_t w, float eps) {
  const HTensor& tx = tensors.at(x);
  const HTensor& tw = tensors.at(w);
  const int64_t dim = tx.shape.back(), rows = tx.numel / dim;
  if (tw.numel != dim || tw.dtype != 0) invalid("rms_norm: weight must be an f32 vector of the last dimension");
  const int dt = act_dtype();
  int64_t o = alloc_pooled(tx.shape);
  ck(eisen_rmsnorm_fwd(stream, operand(tensors[x]), (const float*)tw.data, tensors[o].data, nullptr, rows, dim, eps, dt),
     "rms_norm");
  if (!no_grad) {
    tape.push_back({{x, w}, o, [this, x, w, o, rows, dim, eps, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& gx = tensors[x];
      HTensor& gw = tensors[w];
      ensure_grad(x);
      ensure_grad(w);
      if (!gw.grad_init) { cuck(cudaMemsetAsync(gw.grad, 0, (size_t)dim * 4, stream), "memset"); gw.grad_init = true; }
      void* ws = scratch((size_t)eisen_rmsnorm_bwd_workspace_bytes(rows, dim));
      ck(eisen_rmsnorm_bwd(stream, operand(gx), (const float*)gw.data, to.grad, gx.grad, (float*)gw.grad, ws, rows, dim,
                           eps, dt, gx.grad_init),
         "rms_norm.bwd");
      gx.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/transform.rs:467-612
int64_t Graph::rope(int64_t a, int64_t head_dim) {
  const HTensor& ta = tensors.at(a);
  if (ta.shape.size() != 3) invalid("rope: expects [batch, seq, hidden]");
  const int64_t B = ta.shape[0], S = ta.shape[1], H = ta.shape[2];
  const int dt = act_dtype();
  const float* tab = rope_table(S, head_dim);
  int64_t o = alloc_pooled(ta.shape);
  ck(eisen_rope(stream, operand(tensors[a]), tensors[o].data, tab, B, S, H, head_dim, dt, 0, 0), "rope");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, B, S, H, head_dim, dt, tab]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      ck(eisen_rope(stream, to.grad, ga.grad, tab, B, S, H, head_dim, dt, 1, ga.grad_init), "rope.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/transform.rs:132-326.  idx is an id tensor (alloc_ids) or, as in the reference,
// an f32 tensor of integral values (converted exactly on the host; not a hot path).
int64_t Graph::gather(int64_t w, int64_t idx) {
  const HTensor& tw = tensors.at(w);
  if (tw.shape.size() != 2) invalid("gather: weights must be [vocab, dim]");
  const int64_t vocab = tw.shape[0], dim = tw.shape[1];
  int64_t ids = idx;
  if (tensors.at(idx).dtype != DT_I32) {
    const HTensor& ti = tensors[idx];
    std::vector<float> hf((size_t)ti.numel);
    cuck(cudaMemcpyAsync(hf.data(), ti.data, (size_t)ti.numel * 4, cudaMemcpyDeviceToHost, stream), "D2H(ids)");
    cuck(cudaStreamSynchronize(stream), "sync");
    std::vector<int32_t> hi((size_t)ti.numel);
    for (size_t i = 0; i < hi.size(); ++i) hi[i] = (int32_t)hf[i];
    const std::vector<int64_t> shp = ti.shape;
    ids = alloc_ids(shp, hi.data(), false);
  }
  const int64_t n = tensors[ids].numel;
  std::vector<int64_t> os = tensors[ids].shape;
  os.push_back(dim);
  const int dt = act_dtype();
  int64_t o = alloc_pooled(os);
  ck(eisen_embedding_fwd(stream, operand(tensors[w]), dt, (const int*)tensors[ids].data, tensors[o].data, dt, n, dim,
                         vocab, bad_id_dev),
     "gather");
  if (!no_grad) {
    // The grouping of the positions by id (count, scan, place, order: integer work on the ids alone)
    // runs now, on a side stream beside the first blocks, into a buffer that lives as long as the
    // activations; the backward pass then only adds the gradient rows.  While a step is being
    // captured the grouping stays on the graph's own stream.
    const size_t ws_bytes = (size_t)eisen_embedding_bwd_workspace_bytes(n, vocab);
    const int64_t ws_id = alloc_pooled({(int64_t)((ws_bytes + dsize(dt) - 1) / dsize(dt))});
    tensors[ws_id].constant = true;
    void* ws = tensors[ws_id].data;
    const bool side = !capturing;
    if (side) {
      if (!aux_stream_) {
        cuck(cudaStreamCreateWithFlags(&aux_stream_, cudaStreamNonBlocking), "cudaStreamCreate(aux)");
        cuck(cudaEventCreateWithFlags(&aux_fork_, cudaEventDisableTiming), "cudaEventCreate");
        cuck(cudaEventCreateWithFlags(&aux_join_, cudaEventDisableTiming), "cudaEventCreate");
      }
      cuck(cudaEventRecord(aux_fork_, stream), "cudaEventRecord");
      cuck(cudaStreamWaitEvent(aux_stream_, aux_fork_, 0), "cudaStreamWaitEvent");
      ck(eisen_embedding_bwd_plan(aux_stream_, (const int*)tensors[ids].data, ws, n, vocab), "gather(plan)");
      cuck(cudaEventRecord(aux_join_, aux_stream_), "cudaEventRecord");
      aux_pending_ = true;
    } else {
      ck(eisen_embedding_bwd_plan(stream, (const int*)tensors[ids].data, ws, n, vocab), "gather(plan)");
    }
    tape.push_back({{w, idx}, o, [this, w, o, n, dim, vocab, ws, side]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& gw = tensors[w];
      ensure_grad(w);
      if (gw.grad_dtype != 0) invalid("gather: the table gradient must be f32");
      if (!gw.grad_init) { cuck(cudaMemsetAsync(gw.grad, 0, (size_t)gw.numel * 4, stream), "memset"); gw.grad_init = true; }
      if (side) {
        cuck(cudaStreamWaitEvent(stream, aux_join_, 0), "cudaStreamWaitEvent");
        aux_pending_ = false;
      }
      ck(eisen_embedding_bwd_apply(stream, to.grad, to.grad_dtype, (float*)gw.grad, ws, n, dim, vocab), "gather.bwd");
    }});
  }
  return o;
}

// src/graph/ops/transform.rs:329-409: a physical copy whose backward accumulates
int64_t Graph::reshape(int64_t a, const std::vector<int64_t>& shape) {
  const HTensor& ta = tensors.at(a);
  if (numel_of(shape) != ta.numel) invalid("reshape: element count changes");
  const int dt = act_dtype();
  const int64_t n = ta.numel;
  int64_t o = alloc_pooled(shape);
  ck(eisen_cast(stream, operand(tensors[a]), dt, tensors[o].data, dt, n), "reshape");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, n]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      ck(eisen_accumulate(stream, ga.grad, ga.grad_dtype, to.grad, to.grad_dtype, n, ga.grad_init), "reshape.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/transform.rs:7-129
int64_t Graph::transpose_0213(int64_t a) {
  const HTensor& ta = tensors.at(a);
  if (ta.shape.size() != 4) invalid("transpose_0213: expects a rank-4 tensor");
  const int64_t B = ta.shape[0], S = ta.shape[1], H = ta.shape[2], D = ta.shape[3];
  const int dt = act_dtype();
  int64_t o = alloc_pooled({B, H, S, D});
  ck(eisen_transpose_0213(stream, operand(tensors[a]), tensors[o].data, B, S, H, D, dt, 0), "transpose_0213");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, B, S, H, D, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      // the inverse permutation is the same kernel with S and H exchanged
      ck(eisen_transpose_0213(stream, to.grad, ga.grad, B, H, S, D, dt, ga.grad_init), "transpose_0213.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/gqa.rs:13-196
int64_t Graph::repeat_kv(int64_t a, int64_t repeats) {
  if (repeats == 1) return a;  // gqa.rs:21-23
  const HTensor& ta = tensors.at(a);
  if (ta.shape.size() != 4) invalid("repeat_kv: expects [B, KV, S, D]");
  const int64_t B = ta.shape[0], KV = ta.shape[1], S = ta.shape[2], D = ta.shape[3];
  const int dt = act_dtype();
  int64_t o = alloc_pooled({B, KV * repeats, S, D});
  ck(eisen_repeat_kv_fwd(stream, operand(tensors[a]), tensors[o].data, B, KV, S, D, repeats, dt), "repeat_kv");
  if (!no_grad) {
    tape.push_back({{a}, o, [this, a, o, B, KV, S, D, repeats, dt]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor& ga = tensors[a];
      ensure_grad(a);
      ck(eisen_repeat_kv_bwd(stream, to.grad, ga.grad, B, KV, S, D, repeats, dt, ga.grad_init), "repeat_kv.bwd");
      ga.grad_init = true;
    }});
  }
  return o;
}

// src/graph/ops/attention.rs:7-194: q [BH,M,D], k/v [BH,N,D], forward only (asserts no_grad)
int64_t Graph::flash_attention(int64_t q, int64_t k, int64_t v, float scale, bool causal) {
  if (!no_grad) invalid("flash_attention: forward only, set no_grad (as the reference asserts); training uses attention()");
  const HTensor& tq = tensors.at(q);
  const HTensor& tk = tensors.at(k);
  if (tq.shape.size() != 3 || tk.shape.size() != 3) invalid("flash_attention: expects [batch*heads, seq, head_dim]");
  const int64_t BH = tq.shape[0], S = tq.shape[1], D = tq.shape[2];
  if (tk.shape[1] != S) invalid("flash_attention: query and key lengths must match");
  int64_t o = alloc_pooled({BH, S, D});
  if (precision == Precision::Bf16Mixed) {
    // [BH,S,D] is the [B,S,H,D] layout with H = 1
    ck(eisen_attn_fwd(stream, operand(tensors[q]), operand(tensors[k]), operand(tensors[v]), tensors[o].data, nullptr,
                      BH, S, 1, 1, D, S * D, D, D, S * D, D, D, S * D, D, D, scale, causal, status_dev),
       "flash_attention");
    return o;
  }
  // Fp32: scores -> softmax -> PV with the f32 kernels (exactly the materialised chain)
  float* sc = static_cast<float*>(pool_get((size_t)BH * S * S * 4));
  float* pr = static_cast<float*>(pool_get((size_t)BH * S * S * 4));
  ck(eisen_gemm_f32_strided(stream, (const float*)tensors[q].data, (const float*)tensors[k].data, sc, BH, S, S, D, S * D, D,
                            1, S * D, 1, D, S * S, S, 0),
     "flash.scores");
  ck(eisen_scale_f32(stream, sc, scale, BH * S * S), "flash.scale");
  if (causal) {
    std::vector<float> m((size_t)S * S, 0.0f);
    for (int64_t r = 0; r < S; ++r)
      for (int64_t c = r + 1; c < S; ++c) m[r * S + c] = -1e20f;
    float* md = static_cast<float*>(pool_get((size_t)S * S * 4));
    cuck(cudaMemcpyAsync(md, m.data(), (size_t)S * S * 4, cudaMemcpyHostToDevice, stream), "H2D(mask)");
    ck(eisen_add(stream, sc, md, sc, BH * S * S, S * S, 0), "flash.mask");
    cuck(cudaStreamSynchronize(stream), "sync");
    pool_put(md, (size_t)S * S * 4);
  }
  ck(eisen_softmax_fwd(stream, sc, pr, BH * S, S, 0), "flash.softmax");
  ck(eisen_gemm_f32_strided(stream, pr, (const float*)tensors[v].data, (float*)tensors[o].data, BH, S, D, S, S * S, S, 1,
                            S * D, D, 1, S * D, D, 0),
     "flash.pv");
  pool_put(sc, (size_t)BH * S * S * 4);
  pool_put(pr, (size_t)BH * S * S * 4);
  return o;
}

// Fused causal GQA attention on [B,S,H*D] projections (Bf16Mixed, D in {64,128}); replaces
// reshape/transpose_0213/repeat_kv/bmm/mul/add/softmax/bmm/transpose/reshape of
// src/nn/attention.rs:305-384 and their backward nodes.
int64_t Graph::attention(int64_t q, int64_t k, int64_t v, int64_t Hq, int64_t Hkv, bool causal) {
  if (precision != Precision::Bf16Mixed) invalid("attention: fused attention runs in Bf16Mixed mode");
  const HTensor& tq = tensors.at(q);
  const HTensor& tk = tensors.at(k);
  if (tq.shape.size() != 3) invalid("attention: expects [B, S, heads*head_dim]");
  const int64_t B = tq.shape[0], S = tq.shape[1], D = tq.shape[2] / Hq;
  if (tk.shape[2] != Hkv * D) invalid("attention: k/v width must be kv_heads*head_dim");
  const float scale = 1.0f / std::sqrt((float)D);
  // copies: the allocations below grow `tensors`, which invalidates tq / tk
  const std::vector<int64_t> q_shape = tq.shape;
  const int64_t q_numel = tq.numel;
  const size_t o_bytes = (size_t)q_numel * 2, lse_bytes = (size_t)B * Hq * S * 4;
  const bool slot_ok = attn_stash_slot >= 0 && attn_stash_slot < (int64_t)attn_stash.size();
  const bool replay = attn_stash_mode == 2 && slot_ok && attn_stash[(size_t)attn_stash_slot].o &&
                      attn_stash[(size_t)attn_stash_slot].o_bytes == o_bytes &&
                      attn_stash[(size_t)attn_stash_slot].lse_bytes == lse_bytes;
  // Accuracy of dq / dk in deep models (see eisen_attn_fwd_ex in the header): dS = P (dP - delta) subtracts two
  // numbers that both carry the common component of the value vectors, which is large in deep models.
  //  * v in f32 (Graph::qkv_proj_rope writes it so): the values are centred (v_c = bf16(v - mean over the
  //    sequence)) and forward and backward work on v_c; the second output slot holds the centred output P v_c.
  //  * v in bf16: the second output slot holds the part of the f32 output that the rounding to bf16 drops, and
  //    the backward pass forms delta = dO . (O + O_lo).
  // Against the f32 path the q / k weight gradients of a 16-block model were off by 3.0e-2 with neither and by
  // 2.2e-2 with either; the second form is what runs (v is bf16 unless Graph::center_values is set).
  const bool want_c = !no_grad || (attn_stash_mode == 1 && slot_ok);
  const bool centred = tensors[v].dtype == 0 && precision == Precision::Bf16Mixed;
  int64_t o, lse, o_lo = -1, vc = -1, vmean = -1;
  if (centred) {
    vc = alloc_pooled({B, S, Hkv * D});
    vmean = alloc_pooled_dtype({B, Hkv, D}, 0);
    tensors[vc].constant = tensors[vmean].constant = true;
    ck(eisen_attn_center_values(stream, tensors[v].data, EISEN_F32, tensors[vc].data, (float*)tensors[vmean].data, B, S, Hkv, D,
                                S * Hkv * D, Hkv * D, D),
       "attention(center)");
  }
  if (replay) {
    // the output, its low part and the log-sum-exp of the first forward pass were kept: adopt them, no kernel
    AttnStash& st = attn_stash[(size_t)attn_stash_slot];
    HTensor to_, tl_, tlo_;
    to_.shape = q_shape; to_.numel = q_numel; to_.dtype = to_.grad_dtype = 1; to_.is_pooled = true; to_.data = st.o;
    tl_.shape = {B, Hq, S}; tl_.numel = B * Hq * S; tl_.dtype = tl_.grad_dtype = 0; tl_.is_pooled = true; tl_.data = st.lse;
    tlo_ = to_; tlo_.data = st.o_lo;
    const bool have_lo = st.o_lo != nullptr;
    st = AttnStash();
    o = new_tensor(std::move(to_));
    lse = new_tensor(std::move(tl_));
    if (have_lo) {
      o_lo = new_tensor(std::move(tlo_));
      tensors[o_lo].constant = true;
    }
  } else {
    o = alloc_pooled(q_shape);
    lse = alloc_pooled_dtype({B, Hq, S}, 0);
    if (want_c) {
      o_lo = alloc_pooled(q_shape);
      tensors[o_lo].constant = true;
    }
  }
  tensors[lse].constant = true;
  const int64_t qb = S * Hq * D, qs = Hq * D, kb = S * Hkv * D, ks = Hkv * D;
  // flash convention: 4*B*H*S^2*D forward FLOPs, halved under the causal mask; backward 2.5x
  const double attn_flops = 4.0 * (double)B * (double)Hq * (double)S * (double)S * (double)D * (causal ? 0.5 : 1.0);
  if (!replay) {
    prof_begin(1, attn_flops);
    ck(eisen_attn_fwd_ex(stream, operand(tensors[q]), operand(tensors[k]), centred ? tensors[vc].data : operand(tensors[v]),
                         tensors[o].data, o_lo >= 0 ? tensors[o_lo].data : nullptr,
                         centred ? (const float*)tensors[vmean].data : nullptr, (float*)tensors[lse].data, B, S, Hq, Hkv, D, qb, qs,
                         D, kb, ks, D, qb, qs, D, scale, causal, status_dev),
       "attention");
    prof_end();
    if (attn_stash_mode == 1 && slot_ok) {
      AttnStash& st = attn_stash[(size_t)attn_stash_slot];
      if (st.o) pool_put(st.o, st.o_bytes);
      if (st.o_lo) pool_put(st.o_lo, st.o_bytes);
      if (st.lse) pool_put(st.lse, st.lse_bytes);
      st.o = tensors[o].data; st.lse = tensors[lse].data; st.o_bytes = o_bytes; st.lse_bytes = lse_bytes;
      st.o_lo = o_lo >= 0 ? tensors[o_lo].data : nullptr;
      tensors[o].data_kept = tensors[lse].data_kept = true;  // popped without returning the buffers
      if (o_lo >= 0) tensors[o_lo].data_kept = true;
    }
  }
  if (!no_grad) {
    tape.push_back({{q, k, v}, o, [this, q, k, v, o, o_lo, vc, lse, B, S, Hq, Hkv, D, qb, qs, kb, ks, scale, causal, attn_flops]() {
      OUT_GRAD_OR_RETURN(o);
      HTensor* gt[3] = {&tensors[q], &tensors[k], &tensors[v]};
      void* dst[3];
      void* tmp[3] = {nullptr, nullptr, nullptr};
      const int64_t ids[3] = {q, k, v};
      for (int i = 0; i < 3; ++i) {
        ensure_grad(ids[i]);
        if (gt[i]->grad_dtype != 1) invalid("attention: gradients of q/k/v must be bf16");
        if (gt[i]->grad_init) { tmp[i] = pool_get((size_t)gt[i]->numel * 2); dst[i] = tmp[i]; }
        else dst[i] = gt[i]->grad;
      }
      void* ws = scratch((size_t)eisen_attn_bwd_workspace_bytes(B, S, Hq, Hkv, D));
      // q and k that come from a projection + RoPE op take their gradients rotated back: no separate
      // RoPE backward launch.  Both must be in that form (fresh, or accumulated in it before).
      auto takes_unrotated = [&](const HTensor& t) { return t.unrope_hd == D && (!t.grad_init || t.grad_unrotated); };
      const bool unrope = takes_unrotated(*gt[0]) && takes_unrotated(*gt[1]);
      if (!unrope && (gt[0]->grad_unrotated || gt[1]->grad_unrotated))
        invalid("attention: the gradients of q and k are kept in different forms");
      prof_begin(2, 2.5 * attn_flops);
      if (vc >= 0) {  // centred values: delta from the centred output (held in the second output slot)
        if (o_lo < 0) invalid("attention: the centred output of the forward pass is missing");
        ck(eisen_attn_bwd_ex(stream, operand(*gt[0]), operand(*gt[1]), tensors[vc].data, tensors[o_lo].data, nullptr,
                             (const float*)tensors[lse].data, to.grad, dst[0], dst[1], dst[2], ws, B, S, Hq, Hkv, D, qb, qs, D, kb,
                             ks, D, qb, qs, D, scale, causal, unrope ? rope_table(S, D) : nullptr, status_dev),
           "attention.bwd");
      } else {
        ck(eisen_attn_bwd_ex(stream, operand(*gt[0]), operand(*gt[1]), operand(*gt[2]), to.data,
                             o_lo >= 0 ? tensors[o_lo].data : nullptr, (const float*)tensors[lse].data, to.grad, dst[0], dst[1],
                             dst[2], ws, B, S, Hq, Hkv, D, qb, qs, D, kb, ks, D, qb, qs, D, scale, causal,
                             unrope ? rope_table(S, D) : nullptr, status_dev),
           "attention.bwd");
      }
      if (unrope) gt[0]->grad_unrotated = gt[1]->grad_unrotated = true;
      prof_end();
      for (int i = 0; i < 3; ++i) {
        if (tmp[i]) {
          ck(eisen_accumulate(stream, gt[i]->grad, 1, tmp[i], 1, gt[i]->numel, 1), "attention.bwd(acc)");
          pool_put(tmp[i], (size_t)gt[i]->numel * 2);
        }
        gt[i]->grad_init = true;
      }
    }});
  }
  return o;
}

}  // namespace eisen
