// Graph-level C ABI: opaque handles over Graph / TransformerLM / AdamW (graph.h).  Exceptions
// never cross the boundary: they become status codes plus eisen_last_error().
#include <cstring>

#include "../../../include/eisen_b200.h"
#include "../errors.h"
#include "graph.h"

using namespace eisen;

namespace {

template <class F>
int guarded(F f) {
  try {
    f();
    return 0;
  } catch (const EisenException& e) {
    set_error(e.what());
    return e.code ? e.code : EISEN_ERR_INVALID;
  } catch (const std::out_of_range&) {
    set_error("tensor id out of range");
    return EISEN_ERR_INVALID;
  } catch (const std::bad_alloc&) {
    set_error("host allocation failed");
    return EISEN_ERR_OOM;
  } catch (const std::exception& e) {
    set_error(e.what());
    return EISEN_ERR_INVALID;
  }
}

inline Graph& G(void* g) {
  if (!g) throw EisenException(EISEN_ERR_INVALID, "null graph handle");
  return *static_cast<Graph*>(g);
}
inline std::vector<int64_t> shp(const long long* s, int n) { return std::vector<int64_t>(s, s + n); }

}  // namespace

extern "C" {

int eisen_graph_create(int precision, void* stream, void** out) {
  return guarded([&] {
    if (precision != 0 && precision != 1) throw EisenException(EISEN_ERR_INVALID, "precision must be 0 (Fp32) or 1 (Bf16Mixed)");
    *out = new Graph(precision ? Precision::Bf16Mixed : Precision::Fp32, (cudaStream_t)stream);
  });
}
int eisen_graph_destroy(void* g) {
  return guarded([&] { delete static_cast<Graph*>(g); });
}
int eisen_graph_capture_begin(void* g) {
  return guarded([&] { G(g).capture_begin(); });
}
int eisen_graph_capture_end(void* g, void** exec_out) {
  Graph& gr = G(g);
  int rc = guarded([&] { *exec_out = gr.capture_end(); });
  return rc;
}
int eisen_graph_capture_abort(void* g) {
  return guarded([&] {
    Graph& gr = G(g);
    if (!gr.capturing) return;
    gr.capturing = false;
    cudaGraph_t tmp = nullptr;
    cudaStreamEndCapture(gr.stream, &tmp);
    if (tmp) cudaGraphDestroy(tmp);
    cudaGetLastError();
  });
}
int eisen_graph_replay(void* exec, void* stream) {
  struct CS { cudaGraph_t graph; cudaGraphExec_t exec; };
  if (!exec) return eisen::fail(EISEN_ERR_INVALID, "graph_replay: null handle");
  cudaError_t e = cudaGraphLaunch(static_cast<CS*>(exec)->exec, (cudaStream_t)stream);
  if (e != cudaSuccess) return eisen::fail(EISEN_ERR_CUDA, cudaGetErrorString(e));
  return 0;
}
int eisen_graph_exec_destroy(void* exec) {
  struct CS { cudaGraph_t graph; cudaGraphExec_t exec; };
  if (!exec) return 0;
  CS* cs = static_cast<CS*>(exec);
  if (cs->exec) cudaGraphExecDestroy(cs->exec);
  if (cs->graph) cudaGraphDestroy(cs->graph);
  delete cs;
  return 0;
}
int eisen_graph_selftest_bounded_wait(void* g, long long budget_cycles) {
  return guarded([&] {
    Graph& gr = G(g);
    int rc = eisen_selftest_bounded_wait(gr.stream, gr.status_dev, budget_cycles, nullptr);
    if (rc) throw EisenException(rc, eisen_last_error());
  });
}
int eisen_graph_set_vram_budget(void* g, long long budget_bytes, long long activation_reserve_bytes) {
  return guarded([&] {
    if (budget_bytes < 0 || activation_reserve_bytes < 0) throw EisenException(EISEN_ERR_INVALID, "set_vram_budget: negative size");
    G(g).vram_budget_bytes = (size_t)budget_bytes;
    G(g).activation_reserve_bytes = (size_t)activation_reserve_bytes;
  });
}
int eisen_graph_vram_usage(void* g, long long* used, long long* budget) {
  return guarded([&] {
    if (used) *used = (long long)G(g).current_vram_usage();
    if (budget) *budget = (long long)G(g).vram_budget_bytes;
  });
}
int eisen_graph_plan_streaming(void* g, long long budget_bytes, long long activation_reserve_bytes, const long long* pinned,
                               int n_pinned, int apply, long long* resident_ids, int* n_resident, long long* streamed_ids,
                               int* n_streamed, long long* bytes4) {
  return guarded([&] {
    std::vector<int64_t> pin(pinned, pinned + n_pinned);
    StreamingReport r = apply ? G(g).plan_streaming((size_t)budget_bytes, (size_t)activation_reserve_bytes, pin)
                              : G(g).plan_streaming_layout((size_t)budget_bytes, (size_t)activation_reserve_bytes, pin);
    if (resident_ids) for (size_t i = 0; i < r.resident_param_ids.size(); ++i) resident_ids[i] = r.resident_param_ids[i];
    if (streamed_ids) for (size_t i = 0; i < r.streamed_param_ids.size(); ++i) streamed_ids[i] = r.streamed_param_ids[i];
    if (n_resident) *n_resident = (int)r.resident_param_ids.size();
    if (n_streamed) *n_streamed = (int)r.streamed_param_ids.size();
    if (bytes4) {
      bytes4[0] = r.resident_bytes; bytes4[1] = r.resident_headroom_bytes;
      bytes4[2] = r.streamed_bytes; bytes4[3] = r.streaming_headroom_bytes;
    }
  });
}
int eisen_graph_alloc(void* g, const long long* shape, int ndim, const float* host_data, long long* id_out) {
  return guarded([&] { *id_out = G(g).alloc(shp(shape, ndim), host_data); });
}
int eisen_graph_alloc_ids(void* g, const long long* shape, int ndim, const int* host_ids, long long* id_out) {
  return guarded([&] { *id_out = G(g).alloc_ids(shp(shape, ndim), host_ids, true); });
}
int eisen_graph_alloc_pooled(void* g, const long long* shape, int ndim, long long* id_out) {
  return guarded([&] { *id_out = G(g).alloc_pooled(shp(shape, ndim)); });
}
int eisen_graph_load_tensor_data(void* g, long long id, const float* host, long long n) {
  return guarded([&] { G(g).load_tensor_data(id, host, n); });
}
int eisen_graph_sync_to_cpu(void* g, long long id, float* out) {
  return guarded([&] { G(g).sync_to_cpu(id, out); });
}
int eisen_graph_sync_grad_to_cpu(void* g, long long id, float* out) {
  return guarded([&] { G(g).sync_grad_to_cpu(id, out); });
}
int eisen_graph_shape(void* g, long long id, long long* shape_out, int* ndim_out) {
  return guarded([&] {
    const HTensor& t = G(g).tensors.at(id);
    for (size_t i = 0; i < t.shape.size(); ++i) shape_out[i] = t.shape[i];
    *ndim_out = (int)t.shape.size();
  });
}
int eisen_graph_tensor_ptrs(void* g, long long id, void** data, void** grad, int* dtype, int* grad_dtype) {
  return guarded([&] {
    const HTensor& t = G(g).tensors.at(id);
    if (data) *data = t.data;
    if (grad) *grad = t.grad;
    if (dtype) *dtype = t.dtype;
    if (grad_dtype) *grad_dtype = t.grad_dtype;
  });
}
int eisen_graph_set_no_grad(void* g, int flag) {
  return guarded([&] { G(g).no_grad = flag != 0; });
}
int eisen_graph_get_flags(void* g, int* no_grad, int* skip_forward) {
  return guarded([&] {
    if (no_grad) *no_grad = G(g).no_grad ? 1 : 0;
    if (skip_forward) *skip_forward = G(g).skip_forward ? 1 : 0;
  });
}
int eisen_graph_mark_params(void* g) {
  return guarded([&] { G(g).mark_params(); });
}
int eisen_graph_mark_save_point(void* g, long long* out) {
  return guarded([&] { *out = G(g).mark_save_point(); });
}
int eisen_graph_restore_save_point(void* g, long long sp) {
  return guarded([&] { G(g).restore_save_point(sp); });
}
int eisen_graph_clear_activations(void* g) {
  return guarded([&] { G(g).clear_activations(); });
}
int eisen_graph_tape_clear(void* g) {
  return guarded([&] { G(g).tape.clear(); });
}
int eisen_graph_reinterpret_shape(void* g, long long id, const long long* shape, int ndim) {
  return guarded([&] { G(g).reinterpret_shape(id, shp(shape, ndim)); });
}
int eisen_graph_zero_grad(void* g, long long id) {
  return guarded([&] { G(g).zero_grad(id); });
}
int eisen_graph_backward(void* g, long long loss_id) {
  return guarded([&] { G(g).backward(loss_id); });
}
int eisen_graph_synchronize(void* g) {
  return guarded([&] { G(g).synchronize(); });
}
int eisen_graph_counts(void* g, long long* num_tensors, long long* tape_len, long long* num_params) {
  return guarded([&] {
    Graph& gg = G(g);
    if (num_tensors) *num_tensors = (long long)gg.tensors.size();
    if (tape_len) *tape_len = (long long)gg.tape.size();
    if (num_params) *num_params = gg.num_params;
  });
}
int eisen_graph_pool_stats(void* g, long long* out5) {
  return guarded([&] {
    Graph& gg = G(g);
    out5[0] = (long long)gg.pool_bytes_live;
    out5[1] = (long long)gg.pool_bytes_cached;
    out5[2] = (long long)gg.device_bytes_allocated;
    out5[3] = gg.pool_hits;
    out5[4] = gg.pool_misses;
  });
}
int eisen_graph_param_arena(void* g, void** weights, void** shadow, void** grads, long long* elems) {
  return guarded([&] {
    Graph& gg = G(g);
    if (weights) *weights = gg.arena_w;
    if (shadow) *shadow = gg.arena_shadow;
    if (grads) *grads = gg.arena_g;
    if (elems) *elems = gg.arena_used;
  });
}

#define OP2(name, call) \
  int eisen_graph_##name(void* g, long long a, long long b, long long* out) { return guarded([&] { *out = G(g).call(a, b); }); }
#define OP1(name, call) \
  int eisen_graph_##name(void* g, long long a, long long* out) { return guarded([&] { *out = G(g).call(a); }); }
OP2(add, add)
OP2(mul, mul)
OP1(silu, silu)
OP2(swiglu, swiglu)
OP2(matmul, matmul)
OP2(matmul_trans_b, matmul_trans_b)
OP1(softmax, softmax)
OP2(gather, gather)
OP1(transpose_0213, transpose_0213)
OP2(repeat_kv, repeat_kv)
OP2(rope, rope)

int eisen_graph_matmul_add(void* g, long long a, long long b, long long r, long long* out) {
  return guarded([&] { *out = G(g).matmul_add(a, b, r); });
}
int eisen_graph_bmm(void* g, long long a, long long b, int trans_b, long long* out) {
  return guarded([&] { *out = G(g).bmm(a, b, trans_b != 0); });
}
int eisen_graph_cross_entropy(void* g, long long logits, const long long* targets, long long n, long long* out) {
  return guarded([&] { *out = G(g).cross_entropy(logits, (const int64_t*)targets, n); });
}
int eisen_graph_cross_entropy_masked(void* g, long long logits, const long long* targets, long long n, long long* out) {
  return guarded([&] { *out = G(g).cross_entropy_masked(logits, (const int64_t*)targets, n); });
}
int eisen_graph_lm_head_cross_entropy(void* g, long long h, long long w, long long target_ids, long long n_valid,
                                      int trans_b, long long chunk_rows, long long* out) {
  return guarded([&] {
    *out = G(g).lm_head_cross_entropy(h, w, target_ids, n_valid > 0 ? 1.0f / (float)n_valid : 0.0f, trans_b != 0, chunk_rows);
  });
}
int eisen_graph_rms_norm(void* g, long long x, long long w, float eps, long long* out) {
  return guarded([&] { *out = G(g).rms_norm(x, w, eps); });
}
int eisen_graph_reshape(void* g, long long a, const long long* shape, int ndim, long long* out) {
  return guarded([&] { *out = G(g).reshape(a, shp(shape, ndim)); });
}
int eisen_graph_flash_attention(void* g, long long q, long long k, long long v, float scale, int causal, long long* out) {
  return guarded([&] { *out = G(g).flash_attention(q, k, v, scale, causal != 0); });
}
int eisen_graph_attention(void* g, long long q, long long k, long long v, long long num_heads, long long num_kv_heads,
                          int causal, long long* out) {
  return guarded([&] { *out = G(g).attention(q, k, v, num_heads, num_kv_heads, causal != 0); });
}

// ---- TransformerLM
int eisen_lm_create(void* g, long long vocab, long long hidden, long long heads, long long kv_heads, long long ffn,
                    long long layers, int tie, void** out) {
  return guarded([&] { *out = new TransformerLM(G(g), vocab, hidden, heads, kv_heads, ffn, layers, tie != 0); });
}
int eisen_lm_destroy(void* lm) {
  return guarded([&] { delete static_cast<TransformerLM*>(lm); });
}
int eisen_lm_set_fused(void* lm, int fused) {
  return guarded([&] { static_cast<TransformerLM*>(lm)->fused = fused != 0; });
}
int eisen_lm_set_forward_hook(void* lm, eisen_block_cb before_block, void* user) {
  return guarded([&] {
    TransformerLM* m = static_cast<TransformerLM*>(lm);
    if (before_block) m->before_block = [before_block, user](int64_t l) { before_block((long long)l, user); };
    else m->before_block = nullptr;
  });
}
int eisen_lm_set_keep_attention(void* lm, int keep) {
  return guarded([&] { static_cast<TransformerLM*>(lm)->keep_attention = keep != 0; });
}
int eisen_lm_set_head_fusion(void* lm, int fused, long long chunk_rows) {
  return guarded([&] {
    if (chunk_rows < 0) throw EisenException(EISEN_ERR_INVALID, "lm_set_head_fusion: chunk_rows must be >= 0");
    TransformerLM* m = static_cast<TransformerLM*>(lm);
    m->fused_head = fused != 0;
    m->head_chunk_rows = chunk_rows;
  });
}
int eisen_lm_forward(void* lm, void* g, long long x, long long* out) {
  return guarded([&] { *out = static_cast<TransformerLM*>(lm)->forward(G(g), x); });
}
int eisen_lm_generate(void* lm, void* g, const int* prompt, long long n_prompt, long long max_new_tokens, long long max_context,
                      int kv_cache, int* out_tokens, float* last_logits) {
  return guarded([&] {
    if (!prompt || !out_tokens) throw EisenException(EISEN_ERR_INVALID, "lm_generate: null prompt or output");
    static_cast<TransformerLM*>(lm)->generate(G(g), prompt, n_prompt, max_new_tokens, max_context, kv_cache != 0, out_tokens, last_logits);
  });
}
int eisen_graph_save_weights(void* g, const char* path) {
  return guarded([&] {
    if (!path) throw EisenException(EISEN_ERR_INVALID, "save_weights: null path");
    save_weights(G(g), path);
  });
}
int eisen_graph_load_weights(void* g, const char* path) {
  return guarded([&] {
    if (!path) throw EisenException(EISEN_ERR_INVALID, "load_weights: null path");
    load_weights(G(g), path);
  });
}

int eisen_lm_export_hf(void* lm, void* g, const char* safetensors_path, const char* config_path,
                       long long max_position_embeddings) {
  return guarded([&] {
    if (!lm || !safetensors_path) throw EisenException(EISEN_ERR_INVALID, "lm_export_hf: null argument");
    export_hf(G(g), *static_cast<TransformerLM*>(lm), safetensors_path, config_path, max_position_embeddings);
  });
}

int eisen_lm_params(void* lm, long long* out, int* n) {
  return guarded([&] {
    auto p = static_cast<TransformerLM*>(lm)->params();
    for (size_t i = 0; i < p.size(); ++i) out[i] = p[i];
    *n = (int)p.size();
  });
}
int eisen_lm_train_micro_step(void* lm, void* g, long long x_ids, const long long* targets, long long n_targets,
                              int checkpoint, eisen_block_cb after_block, void* user, long long* loss_id) {
  return guarded([&] {
    std::function<void(int64_t)> cb;
    if (after_block) cb = [after_block, user](int64_t l) { after_block((long long)l, user); };
    *loss_id = static_cast<TransformerLM*>(lm)->train_micro_step(G(g), x_ids, (const int64_t*)targets, n_targets,
                                                                 checkpoint != 0, cb);
  });
}

int eisen_lm_train_micro_step_dev(void* lm, void* g, long long x_ids, long long target_ids, long long n_valid,
                                  int checkpoint, eisen_block_cb after_block, void* user, long long* loss_id) {
  return guarded([&] {
    std::function<void(int64_t)> cb;
    if (after_block) cb = [after_block, user](int64_t l) { after_block((long long)l, user); };
    *loss_id = static_cast<TransformerLM*>(lm)->train_micro_step_dev(G(g), x_ids, target_ids, n_valid, checkpoint != 0, cb);
  });
}
int eisen_graph_prof_enable(void* g, int on) {
  return guarded([&] { G(g).prof_on = on != 0; });
}
int eisen_graph_prof_read(void* g, double* out9) {
  return guarded([&] { G(g).prof_read(out9); });
}

// ---- AdamW
int eisen_optim_create(void* g, const long long* params, int n, float lr, void** out) {
  return guarded([&] { *out = new AdamW(G(g), std::vector<int64_t>(params, params + n), lr); });
}
int eisen_optim_destroy(void* opt) {
  return guarded([&] { delete static_cast<AdamW*>(opt); });
}
int eisen_optim_config(void* opt, float lr, float beta1, float beta2, float eps, float weight_decay) {
  return guarded([&] {
    AdamW& o = *static_cast<AdamW*>(opt);
    o.lr = lr; o.beta1 = beta1; o.beta2 = beta2; o.eps = eps; o.weight_decay = weight_decay;
  });
}
int eisen_optim_zero_grad(void* opt) {
  return guarded([&] { static_cast<AdamW*>(opt)->zero_grad(); });
}
int eisen_optim_clip_grad_norm(void* opt, float max_norm, float* norm_out, float* coef_out) {
  return guarded([&] {
    float coef = 1.0f;
    float n = static_cast<AdamW*>(opt)->clip_grad_norm(max_norm, &coef);
    if (norm_out) *norm_out = n;
    if (coef_out) *coef_out = coef;
  });
}
int eisen_optim_step(void* opt) {
  return guarded([&] { static_cast<AdamW*>(opt)->step(); });
}
int eisen_optim_step_fused(void* opt, float max_norm, float grad_scale) {
  return guarded([&] { static_cast<AdamW*>(opt)->step_fused(max_norm, grad_scale); });
}
int eisen_optim_advance(void* opt) {
  return guarded([&] { static_cast<AdamW*>(opt)->advance(); });
}
int eisen_optim_save_state(void* opt, const char* path) {
  return guarded([&] { static_cast<AdamW*>(opt)->save_state(path); });
}
int eisen_optim_load_state(void* opt, const char* path) {
  return guarded([&] { static_cast<AdamW*>(opt)->load_state(path); });
}
int eisen_optim_create_sharded(void* g, const long long* params, int n, float lr, const long long* piece_lo,
                               const long long* piece_hi, int n_pieces, void** out) {
  return guarded([&] {
    std::vector<std::pair<int64_t, int64_t>> pieces;
    for (int i = 0; i < n_pieces; ++i) pieces.emplace_back(piece_lo[i], piece_hi[i]);
    *out = new AdamW(G(g), std::vector<int64_t>(params, params + n), lr, std::move(pieces));
  });
}
int eisen_optim_begin_step(void* opt) {
  return guarded([&] { static_cast<AdamW*>(opt)->begin_step(); });
}
int eisen_optim_sumsq_piece(void* opt, int piece, int accumulate, void* stream) {
  return guarded([&] {
    AdamW* o = static_cast<AdamW*>(opt);
    o->sumsq_piece((size_t)piece, accumulate != 0, stream ? (cudaStream_t)stream : o->g.stream);
  });
}
int eisen_optim_step_piece(void* opt, int piece, float max_norm, float grad_scale) {
  return guarded([&] { static_cast<AdamW*>(opt)->step_piece((size_t)piece, max_norm, grad_scale); });
}
int eisen_optim_step_piece_on(void* opt, int piece, float max_norm, float grad_scale, void* stream, int zero_grads) {
  return guarded([&] {
    static_cast<AdamW*>(opt)->step_piece((size_t)piece, max_norm, grad_scale, (cudaStream_t)stream, zero_grads != 0);
  });
}
int eisen_optim_sumsq_ptr(void* opt, void** out) {
  return guarded([&] { *out = static_cast<AdamW*>(opt)->sumsq_dev; });
}
int eisen_optim_is_flat(void* opt, int* flat) {
  return guarded([&] { *flat = static_cast<AdamW*>(opt)->flat ? 1 : 0; });
}

}  // extern "C"
