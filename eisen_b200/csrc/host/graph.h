// Host-side mirror of the reference's Graph / Tape / Tensor (src/graph/mod.rs:56-78,
// src/tape.rs:3-12, src/tensor.rs:19-44) with the `Device::Gpu` arms of its ops rebuilt on the
// kernels of this library.  Tensor ids are indices into `tensors`, ops run the forward at once
// and push a tape node (unless no_grad), `backward` walks the tape in reverse.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace eisen {

enum class Precision : int { Fp32 = 0, Bf16Mixed = 1 };  // src/graph/mod.rs PrecisionMode
constexpr int DT_I32 = 2;                                 // token-id tensors (device int32)

struct EisenException : std::runtime_error {
  int code;
  EisenException(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

struct HTensor {
  std::vector<int64_t> shape;
  int64_t numel = 0;
  int dtype = 0;           // DT_F32 / DT_BF16 / DT_I32 of `data`
  void* data = nullptr;
  void* shadow = nullptr;  // bf16 copy of an f32 parameter (Bf16Mixed), refreshed by AdamW
  void* grad = nullptr;
  int grad_dtype = 0;
  bool grad_init = false;  // false: grad holds garbage and stands for zero; first writer overwrites
  bool is_pooled = false;  // activation: buffers return to the pool on restore_save_point
  bool data_kept = false;  // pooled tensor whose data buffer was handed to Graph::attn_stash: not returned to the pool
  bool owns_data = false;  // free with cudaFree on destruction (non-pooled, non-arena)
  bool owns_grad = false;
  bool is_param = false;
  // Parameter homed in page-locked host memory that the GPU can address (a "streamed" parameter of
  // the reference, src/graph/memory.rs:125-170): data, shadow and grad are host pointers; kernels
  // that read rows or elements use them in place over PCIe, GEMM operands are staged on the device.
  bool host_homed = false;
  bool grad_is_ones = false;  // the gradient was seeded with ones by backward() and not written since
  // Output of a projection + RoPE op that can take its gradient already rotated back (head_dim; 0 = no):
  // the fused attention backward then writes dq / dk in that form and sets grad_unrotated.
  int64_t unrope_hd = 0;
  bool grad_unrotated = false;
  bool constant = false;   // no gradient is ever formed (masks, scale tensors, ids)
  std::string name;
};

// src/graph/memory.rs:7-14
struct StreamingReport {
  std::vector<int64_t> resident_param_ids, streamed_param_ids;
  int64_t resident_bytes = 0, resident_headroom_bytes = 0, streamed_bytes = 0, streaming_headroom_bytes = 0;
};

struct HNode {
  std::vector<int64_t> inputs;
  int64_t output;
  std::function<void()> backward;
};

class Graph {
 public:
  Graph(Precision prec, cudaStream_t stream);
  ~Graph();

  // ---- storage (src/graph/mod.rs: alloc, alloc_pooled 437-556, load_tensor_data 368-430)
  int64_t alloc(const std::vector<int64_t>& shape, const float* host_data);  // f32 leaf / parameter
  int64_t alloc_ids(const std::vector<int64_t>& shape, const int32_t* host_ids, bool host_is_pinned_async);
  int64_t alloc_pooled(const std::vector<int64_t>& shape);                   // activation dtype
  int64_t alloc_pooled_dtype(const std::vector<int64_t>& shape, int dtype);
  void load_tensor_data(int64_t id, const float* host, int64_t n);
  void sync_to_cpu(int64_t id, float* out);       // Tensor::sync_to_cpu
  void sync_grad_to_cpu(int64_t id, float* out);  // Graph::sync_grad_to_cpu
  void reserve_param_arena(int64_t total_elems);  // parameters allocated afterwards share flat buffers
  void name_tensor(int64_t id, const std::string& n) { tensors.at(id).name = n; }

  // ---- graph state (src/graph/mod.rs:328-365, 432-435)
  void mark_params() { num_params = (int64_t)tensors.size(); }
  int64_t mark_save_point() const { return (int64_t)tensors.size(); }
  void restore_save_point(int64_t sp);
  void clear_activations();
  void reinterpret_shape(int64_t id, const std::vector<int64_t>& shape);
  void zero_grad(int64_t id);
  void backward(int64_t loss_id);
  void backward_from(int64_t tape_begin);  // walks nodes [tape_begin, end) in reverse, no seeding
  void seed_grad_ones(int64_t id);
  void synchronize();
  void check_status();                      // raises if a kernel recorded a fault
  // CUDA-graph capture of everything enqueued on the graph's stream between the two calls (a whole
  // training step of a small model is hundreds of launches of a few microseconds: launch-bound).
  // The captured work must allocate nothing and never wait on the host: run the same step eagerly
  // first so that the pool, the scratch buffers and the RoPE tables are warm.  The executable
  // graph replays the captured launches with the captured pointers.
  void capture_begin();
  void* capture_end();                      // -> handle for graph_replay / graph_exec_destroy
  bool capturing = false;

  // ---- ops (src/graph/ops/*.rs)
  int64_t add(int64_t a, int64_t b);
  int64_t mul(int64_t a, int64_t b);
  int64_t silu(int64_t a);
  int64_t swiglu(int64_t gate, int64_t up);
  int64_t gate_up_swiglu(int64_t x, int64_t wg, int64_t wu);
  int64_t matmul_rope(int64_t a, int64_t b, int64_t head_dim);
  // q = rope(x Wq), k = rope(x Wk), v = x Wv as one tape entry (out3 = {q, k, v})
  void qkv_proj_rope(int64_t x, int64_t wq, int64_t wk, int64_t wv, int64_t head_dim, int64_t out3[3]);
  int64_t matmul(int64_t a, int64_t b);
  int64_t matmul_trans_b(int64_t a, int64_t b);
  // r + a b in one launch (Bf16Mixed): the residual add done in the projection's epilogue
  int64_t matmul_add(int64_t a, int64_t b, int64_t r);
  int64_t bmm(int64_t a, int64_t b, bool trans_b);
  int64_t softmax(int64_t a);
  int64_t cross_entropy(int64_t logits, const int64_t* targets, int64_t n);
  int64_t cross_entropy_masked(int64_t logits, const int64_t* targets, int64_t n);
  int64_t rms_norm(int64_t x, int64_t w, float eps);
  int64_t rope(int64_t a, int64_t head_dim);
  int64_t gather(int64_t w, int64_t idx);
  int64_t reshape(int64_t a, const std::vector<int64_t>& shape);
  int64_t transpose_0213(int64_t a);
  int64_t repeat_kv(int64_t a, int64_t repeats);
  int64_t flash_attention(int64_t q, int64_t k, int64_t v, float scale, bool causal);  // [BH,S,D], forward only
  // fused GQA attention on the projections' [B,S,H*D] outputs, with backward
  int64_t attention(int64_t q, int64_t k, int64_t v, int64_t num_heads, int64_t num_kv_heads, bool causal);

  // ---- VRAM budget and parameter streaming (src/graph/mod.rs:283-288, src/graph/memory.rs:64-266)
  // Budget in bytes for everything this graph allocates on the device (0 = none).  Read from
  // EISEN_VRAM_BUDGET_MB when the graph is created, like the reference.  Activation allocations that
  // would exceed it first drop the cached pool buffers and then fail with EISEN_ERR_OOM.
  size_t vram_budget_bytes = 0;
  size_t activation_reserve_bytes = 64u << 20;  // EISEN_ACTIVATION_RESERVE_MB, default 64
  size_t current_vram_usage() const { return device_bytes_allocated; }
  // While set, parameters created by alloc() are homed in host memory (TransformerLM sets it around
  // the 2-D block weights when a budget is in force, src/nn/transformer.rs:92-101).
  bool home_params_on_host = false;
  // The planning arithmetic of plan_streaming only (no tensor is moved): which parameters fit the
  // budget at 16 bytes per element (weight, gradient, two moments), the rest is streamed.
  StreamingReport plan_streaming_layout(size_t vram_budget, size_t activation_reserve, const std::vector<int64_t>& pinned) const;
  // Plans and then re-homes: resident parameters are moved to device memory, streamed ones to host memory.
  StreamingReport plan_streaming(size_t vram_budget, size_t activation_reserve, const std::vector<int64_t>& pinned);
  void move_param_to_host(int64_t id);
  void move_param_to_device(int64_t id);
  // Device copy of a weight for use as a GEMM operand: the tensor's own buffer, or for a host-homed
  // parameter a slot of the staging ring filled on the copy stream (prefetch_weight starts that copy
  // early, at the latest it is started here).  The compute stream is made to wait for the copy.
  const void* weight_operand(int64_t id);
  void prefetch_weight(int64_t id);
  void invalidate_staged_weights() { ++weight_generation_; }

  // Selective recompute for per-block checkpointing: with attn_stash_mode == 1 the fused attention
  // op hands its output and log-sum-exp buffers to attn_stash[attn_stash_slot] instead of the pool
  // when its tensors are popped; with mode 2 it adopts the stashed buffers and skips its forward
  // kernel (the block re-run for the backward pass then recomputes everything except attention).
  struct AttnStash { void* o = nullptr; void* o_lo = nullptr; void* lse = nullptr; size_t o_bytes = 0, lse_bytes = 0; };
  std::vector<AttnStash> attn_stash;
  int attn_stash_mode = 0;
  int64_t attn_stash_slot = -1;
  void release_attn_stash();  // returns every stashed buffer to the pool

  // ---- helpers used by modules / optimizer
  int act_dtype() const { return precision == Precision::Bf16Mixed ? 1 : 0; }
  void* pool_get(size_t bytes);
  void pool_put(void* p, size_t bytes);
  void* scratch(size_t bytes);  // grow-only scratch buffer valid until the next scratch() call
  void ensure_grad(int64_t id);
  const float* rope_table(int64_t seq_len, int64_t head_dim);
  int64_t ce_impl(int64_t logits, const int64_t* targets, int64_t n, bool masked, float normalizer);
  int64_t ce_device(int64_t logits, int64_t target_ids, float normalizer);  // targets already on the device
  // LM head and cross-entropy as one op: loss = CE(h W, targets) with W [k, vocab] (or, trans_b,
  // the tied table [vocab, k]).  The token rows are worked through in chunks of chunk_rows (0 =
  // all at once): logits of a chunk -> loss and dlogits in place (one read, one write) -> dH rows
  // and dW, so only a [chunk_rows, vocab] slab of logits ever exists.  The gradients are formed
  // during the forward with the loss gradient taken as 1: the result must be the tensor that
  // backward() starts from (checked there).  Under no_grad only the loss is computed.
  int64_t lm_head_cross_entropy(int64_t h, int64_t w, int64_t target_ids, float normalizer, bool trans_b,
                                int64_t chunk_rows);

  // event-based timing of the tensor-core kernels (class 0 GEMM, 1 attention fwd, 2 attention bwd)
  bool prof_on = false;
  struct ProfRec { cudaEvent_t a, b; double flops; int cls; };
  std::vector<ProfRec> prof_recs;
  std::vector<cudaEvent_t> prof_free;
  void prof_begin(int cls, double flops);
  void prof_end();
  void prof_read(double* out9);
  const void* operand(const HTensor& t) const;  // bf16 shadow of an f32 parameter in Bf16Mixed

  std::vector<HTensor> tensors;
  std::vector<HNode> tape;
  bool no_grad = false;
  // When set, matmul and add record their tape node and allocate their output but do not run the
  // forward kernel.  Used while a checkpointed block is re-run for its backward pass: the values of
  // the last projection and of the last residual add are read by no backward node.
  bool skip_forward = false;
  // Off by default and set by nobody in this library: qkv_proj_rope then writes the value projection in f32 and
  // attention centres it before rounding (see Graph::attention).  Measured on a 16-block model: no better than
  // the default (the low part of the attention output handed to the backward pass), at 1 ms more per step.
  bool center_values = false;
  int64_t num_params = 0;
  Precision precision;
  cudaStream_t stream;
  int* status_dev = nullptr;  // fault word of the tensor-core kernels
  int* bad_id_dev = nullptr;

  // flat parameter arena (f32 weights | bf16 shadow | f32 grads), element offsets
  float* arena_w = nullptr;
  void* arena_shadow = nullptr;
  float* arena_g = nullptr;
  int64_t arena_cap = 0, arena_used = 0;

  size_t pool_bytes_cached = 0, pool_bytes_live = 0, device_bytes_allocated = 0;
  int64_t pool_hits = 0, pool_misses = 0;

 private:
  std::unordered_map<size_t, std::vector<void*>> pool_;
  void* scratch_ = nullptr;
  size_t scratch_bytes_ = 0;
  std::unordered_map<int64_t, float*> rope_tables_;
  // staging ring for host-homed GEMM operands
  struct StageSlot { void* buf = nullptr; int64_t id = -1; uint64_t generation = 0; cudaEvent_t ready = nullptr; };
  std::vector<StageSlot> stage_;
  size_t stage_slot_bytes_ = 0;
  size_t stage_next_ = 0;
  uint64_t weight_generation_ = 1;
  cudaStream_t copy_stream_ = nullptr;
  // side stream for work that depends on the token ids only (the grouping of the embedding backward)
  cudaStream_t aux_stream_ = nullptr;
  cudaEvent_t aux_fork_ = nullptr, aux_join_ = nullptr;
  bool aux_pending_ = false;  // side-stream work the graph's stream has not waited for yet
  cudaEvent_t compute_mark_ = nullptr;
  void ensure_stage(size_t bytes);
  StageSlot* stage_weight(int64_t id);
  int64_t new_tensor(HTensor&& t);
  void free_tensor(HTensor& t);
};

// Sets a graph mode flag (no_grad, skip_forward) for a scope and restores the previous value on
// every way out, so an exception inside a block forward cannot leave the graph in that mode.
struct FlagGuard {
  bool& flag;
  bool saved;
  FlagGuard(bool& f, bool value) : flag(f), saved(f) { flag = value; }
  ~FlagGuard() { flag = saved; }
  FlagGuard(const FlagGuard&) = delete;
  FlagGuard& operator=(const FlagGuard&) = delete;
};

// ---------------------------------------------------------------------------------------
// modules (src/nn/*.rs)
// ---------------------------------------------------------------------------------------
struct BlockParams {
  int64_t norm1, q, k, v, o, norm2, gate, up, down;
};

class TransformerLM {
 public:
  // src/nn/transformer.rs:81-122
  TransformerLM(Graph& g, int64_t vocab, int64_t hidden, int64_t heads, int64_t kv_heads, int64_t ffn,
                int64_t layers, bool tie);
  int64_t forward(Graph& g, int64_t x_ids);                       // :184-196
  // skip_dead_tail: leave out the forward kernels whose results no backward node reads
  // kv_out (optional): receives the ids of the rotated key projection and of the value projection,
  // [B, S, kv_heads * head_dim] each (what a KV cache keeps)
  int64_t block_forward(Graph& g, const BlockParams& b, int64_t x, bool skip_dead_tail = false,
                        std::pair<int64_t, int64_t>* kv_out = nullptr);  // :32-49
  int64_t gqa_forward(Graph& g, const BlockParams& b, int64_t x, bool causal, int64_t residual = -1,
                      std::pair<int64_t, int64_t>* kv_out = nullptr);  // attention.rs:289-388
  // Greedy generation as in examples/train_llm.rs:560-584 (argmax of the last position's logits,
  // context window max_context).  kv_cache = false runs that loop as the reference does, the
  // whole context through forward() for every token.  kv_cache = true keeps every layer's rotated
  // keys and values: the prompt is run once, each further token is one row through the
  // projections plus eisen_attn_decode over the cache (README.md:94 lists this as future work);
  // it needs n_prompt + max_new <= max_context, because a sliding window re-positions every token.
  // out_tokens receives max_new tokens; last_logits (may be null) the [vocab] logits behind the last one.
  void generate(Graph& g, const int32_t* prompt, int64_t n_prompt, int64_t max_new, int64_t max_context, bool kv_cache,
                int32_t* out_tokens, float* last_logits);
  std::vector<int64_t> params() const;                            // :198-210
  // starts the host-to-device copies of block l's host-homed weights (no-op for resident ones)
  void prefetch_block(Graph& g, int64_t l) const;
  // One micro-step: forward, loss (masked cross-entropy over [B*S] targets), backward.
  // checkpoint = true keeps only block inputs in the forward and re-runs each block under a
  // save point during the backward (the primitives of src/graph/mod.rs:332-365).
  // after_block(l) is called when the gradients of block l (and, with l == layers, of the
  // final norm / head; with l == -1, of the embedding) are complete.
  int64_t train_micro_step(Graph& g, int64_t x_ids, const int64_t* targets, int64_t n_targets, bool checkpoint,
                           const std::function<void(int64_t)>& after_block);
  int64_t train_micro_step_dev(Graph& g, int64_t x_ids, int64_t target_ids, int64_t n_valid, bool checkpoint,
                               const std::function<void(int64_t)>& after_block);
  int64_t vocab, hidden, heads, kv_heads, ffn, layers;
  bool tie;
  bool fused = true;  // fused attention / SwiGLU ops (always the reference chain in Fp32 mode when false)
  // train_micro_step: head projection and cross-entropy as one op (Graph::lm_head_cross_entropy)
  // working through head_chunk_rows token rows at a time (0 = all rows at once)
  // per-block checkpointing keeps the attention output and log-sum-exp of every block (66 MB per
  // block at 8 x 2048 tokens, d 2048) and does not run the attention forward again in the backward pass
  bool keep_attention = false;
  // called in train_micro_step before the forward pass first touches the parameters of block l
  // (l == -1: embedding, l == layers: final norm and head); a sharded data-parallel step uses it to
  // wait for the all-gather of exactly those weights instead of for all of them up front
  std::function<void(int64_t)> before_block;
  bool fused_head = true;
  int64_t head_chunk_rows = 0;
  int64_t emb, norm_f, head;
  std::vector<BlockParams> blocks;
};

// examples/export_hf_pipeline.rs, src/tools/huggingface.rs: model.safetensors + config.json (export_hf.cpp)
void export_hf(Graph& g, const TransformerLM& lm, const char* safetensors_path, const char* config_path,
               int64_t max_position_embeddings);

// examples/train_llm.rs:92-105: weights-only checkpoint (all parameter tensors in id order, f32), and its inverse
void save_weights(Graph& g, const char* path);
void load_weights(Graph& g, const char* path);

// src/nn/optim.rs
class AdamW {
 public:
  AdamW(Graph& g, std::vector<int64_t> params, float lr);
  ~AdamW();
  void zero_grad();                                    // :207-245
  float clip_grad_norm(float max_norm, float* coef);   // :250-321 (host-visible norm, one 8-byte read-back)
  void step();                                         // :334-481
  // no host synchronisation: norm and clip coefficient stay on the device; grad_scale folds the
  // data-parallel 1/world factor
  void step_fused(float max_norm, float grad_scale);
  // Sharded state (ZeRO-1): this rank keeps moments only for `pieces` (element ranges of the flat
  // arena) and updates only those; the other ranks' pieces arrive through the exchange.
  AdamW(Graph& g, std::vector<int64_t> params, float lr, std::vector<std::pair<int64_t, int64_t>> pieces);
  void begin_step() { t += 1; }                       // once per optimizer step, before step_piece
  void sumsq_piece(size_t i, bool accumulate, cudaStream_t s);   // sumsq_dev (op)= sum g^2 over piece i
  void step_piece(size_t i, float max_norm, float grad_scale, cudaStream_t s = nullptr, bool zero_grads = false);   // clip coefficient from sumsq_dev when max_norm > 0
  // Optimizer state of a checkpoint (the reference saves weights only and lists this as future
  // work, README.md:88): step count t, hyper-parameters and the moments of the ranges this object owns.
  void save_state(const char* path);
  void load_state(const char* path);
  int64_t state_elems() const;
  std::vector<std::pair<int64_t, int64_t>> pieces;
  std::vector<int64_t> piece_state_off;  // offset of each piece's moments in m / v
  float lr, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0.01f;
  int64_t t = 0;
  Graph& g;
  std::vector<int64_t> params;
  bool flat = false;  // parameters cover the arena: one launch
  float* m = nullptr;
  float* v = nullptr;
  std::vector<int64_t> offsets;  // per-parameter offsets into m / v when not flat
  // not flat: where each parameter's moments live; a host-homed parameter keeps them in host memory
  // (the reference's streamed parameters are updated by its CPU arm, src/nn/optim.rs:523-543)
  std::vector<float*> m_ptr, v_ptr;
  std::vector<float*> host_moments;  // page-locked buffers owned by this optimizer
  // step-dependent scalars of a captured step: {lr, bc1, bc2, -} in page-locked host memory, copied to
  // the device by a node of the captured graph
  float* hyper_host = nullptr;
  float* hyper_dev = nullptr;
  void advance();
  int64_t total = 0;
  double* sumsq_dev = nullptr;
  void* sumsq_ws = nullptr;

 private:
  void launch(float grad_scale, const double* sumsq, float max_norm);
};

}  // namespace eisen
