// Modules and optimizer of the training step: TransformerLM (src/nn/transformer.rs),
// GroupedQueryAttention (src/nn/attention.rs:251-404), Linear / Embedding / RMSNorm
// (src/nn/linear.rs, embedding.rs, rmsnorm.rs) and AdamW (src/nn/optim.rs), on the Graph of
// graph.h.  Parameter ids, creation order and params() order follow the reference.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "../../../include/eisen_b200.h"
#include "graph.h"

namespace eisen {

namespace {

void ck(int rc, const char* what) {
  if (rc != 0) throw EisenException(rc, std::string(what) + ": " + eisen_last_error());
}
void cuck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw EisenException(EISEN_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// src/nn/linear.rs:10-49: LCG + Box-Muller, std 0.02; the seed restarts at 42 for every layer
std::vector<float> linear_init(size_t n) {
  std::vector<float> w(n);
  uint32_t seed = 42;
  const float umax = (float)UINT32_MAX;
  for (size_t i = 0; i < n; ++i) {
    float u1 = std::min((float)seed / umax + 1e-7f, 1.0f - 1e-7f);
    seed = seed * 1664525u + 1013904223u;
    float u2 = std::min(std::max((float)seed / umax, 1e-7f), 1.0f - 1e-7f);
    seed = seed * 1664525u + 1013904223u;
    float mag = std::sqrt(-2.0f * std::log(u1));
    w[i] = mag * std::cos(2.0f * 3.14159265358979323846f * u2) * 0.02f;
  }
  return w;
}
// src/nn/embedding.rs:9-32
std::vector<float> embedding_init(size_t n) {
  std::vector<float> w(n);
  uint32_t seed = 84;
  const float umax = (float)UINT32_MAX;
  for (size_t i = 0; i < n; ++i) {
    seed = seed * 1664525u + 1013904223u;
    w[i] = (((float)seed / umax) * 2.0f - 1.0f) * 0.02f;
  }
  return w;
}

int64_t pad64(int64_t n) { return (n + 63) / 64 * 64; }

int64_t linear_new(Graph& g, int64_t in, int64_t out, std::vector<float>& cache) {
  const size_t n = (size_t)in * out;
  if (cache.size() < n) cache = linear_init(n);  // every layer draws the same stream: a prefix is enough
  return g.alloc({in, out}, cache.data());
}
int64_t norm_new(Graph& g, int64_t d) {
  std::vector<float> ones((size_t)d, 1.0f);
  return g.alloc({d}, ones.data());
}

// src/nn/linear.rs:53-95 (no bias on this path)
int64_t linear_fwd(Graph& g, int64_t x, int64_t w) {
  const std::vector<int64_t> xs = g.tensors.at(x).shape;
  int64_t o = g.matmul(x, w);
  if (xs.size() == 3) g.reinterpret_shape(o, {xs[0], xs[1], g.tensors[w].shape[1]});
  return o;
}

}  // namespace

TransformerLM::TransformerLM(Graph& g, int64_t vocab_, int64_t hidden_, int64_t heads_, int64_t kv_heads_,
                             int64_t ffn_, int64_t layers_, bool tie_)
    : vocab(vocab_), hidden(hidden_), heads(heads_), kv_heads(kv_heads_), ffn(ffn_), layers(layers_), tie(tie_) {
  if (hidden % heads) throw EisenException(EISEN_ERR_INVALID, "hidden_dim must be cleanly divisible by num_heads");
  if (heads % kv_heads) throw EisenException(EISEN_ERR_INVALID, "num_heads must be divisible by num_kv_heads");
  const int64_t hd = hidden / heads, kvd = kv_heads * hd;
  // With a VRAM budget in force the 2-D block weights start out in host memory, as the reference
  // demotes them while it builds the model (src/nn/transformer.rs:92-101); Graph::plan_streaming
  // decides afterwards which of them move to the device.  Only embedding, norms and head share the arena.
  const bool budgeted = g.vram_budget_bytes > 0;
  if (!g.arena_w && g.num_params == 0) {
    int64_t total = pad64(vocab * hidden) + pad64(hidden) + (tie ? 0 : pad64(hidden * vocab));
    total += layers * 2 * pad64(hidden);
    if (!budgeted) total += layers * (2 * pad64(hidden * hidden) + 2 * pad64(hidden * kvd) + 3 * pad64(hidden * ffn));
    g.reserve_param_arena(total);
  }
  auto block_linear = [&](int64_t in, int64_t out, std::vector<float>& c) {
    FlagGuard host(g.home_params_on_host, budgeted);
    return linear_new(g, in, out, c);
  };
  std::vector<float> cache;
  {
    std::vector<float> e = embedding_init((size_t)vocab * hidden);
    emb = g.alloc({vocab, hidden}, e.data());
  }
  // creation order of TransformerBlock::new (src/nn/transformer.rs:19-29)
  for (int64_t l = 0; l < layers; ++l) {
    BlockParams b;
    b.norm1 = norm_new(g, hidden);
    b.q = block_linear(hidden, hidden, cache);
    b.k = block_linear(hidden, kvd, cache);
    b.v = block_linear(hidden, kvd, cache);
    b.o = block_linear(hidden, hidden, cache);
    b.norm2 = norm_new(g, hidden);
    b.gate = block_linear(hidden, ffn, cache);
    b.up = block_linear(hidden, ffn, cache);
    b.down = block_linear(ffn, hidden, cache);
    blocks.push_back(b);
  }
  norm_f = norm_new(g, hidden);
  head = tie ? emb : linear_new(g, hidden, vocab, cache);
  fused = (g.precision == Precision::Bf16Mixed) && (hd == 64 || hd == 128);
}

std::vector<int64_t> TransformerLM::params() const {
  std::vector<int64_t> p{emb};
  for (const BlockParams& b : blocks) {
    p.insert(p.end(), {b.norm1, b.q, b.k, b.v, b.o, b.norm2, b.up, b.down, b.gate});
  }
  p.push_back(norm_f);
  if (!tie) p.push_back(head);
  return p;
}

void TransformerLM::prefetch_block(Graph& g, int64_t l) const {
  if (l < 0 || l >= layers) return;
  const BlockParams& b = blocks[(size_t)l];
  for (int64_t id : {b.q, b.k, b.v, b.o, b.gate, b.up, b.down}) g.prefetch_weight(id);
}

int64_t TransformerLM::gqa_forward(Graph& g, const BlockParams& b, int64_t x, bool causal, int64_t residual,
                                   std::pair<int64_t, int64_t>* kv_out) {
  const std::vector<int64_t> xs = g.tensors.at(x).shape;
  if (xs.size() != 3) throw EisenException(EISEN_ERR_INVALID, "GQA requires [Batch, Seq, Dim]");
  const int64_t B = xs[0], S = xs[1], hd = hidden / heads;
  int64_t qr, kr, v;
  if (fused) {  // the three projections, RoPE on q and k, as one tape entry
    int64_t out3[3];
    g.qkv_proj_rope(x, b.q, b.k, b.v, hd, out3);
    qr = out3[0]; kr = out3[1]; v = out3[2];
  } else {
    int64_t q = linear_fwd(g, x, b.q), k = linear_fwd(g, x, b.k);
    qr = g.rope(q, hd);
    kr = g.rope(k, hd);
    v = linear_fwd(g, x, b.v);
  }
  if (kv_out) *kv_out = {kr, v};
  int64_t ctx2;
  if (fused) {
    ctx2 = g.attention(qr, kr, v, heads, kv_heads, causal);
  } else {
    // the reference chain, op for op (src/nn/attention.rs:305-384)
    int64_t q4 = g.reshape(qr, {B, S, heads, hd});
    int64_t k4 = g.reshape(kr, {B, S, kv_heads, hd});
    int64_t v4 = g.reshape(v, {B, S, kv_heads, hd});
    int64_t qt = g.transpose_0213(q4), kt = g.transpose_0213(k4), vt = g.transpose_0213(v4);
    const int64_t rep = heads / kv_heads;
    int64_t krep = g.repeat_kv(kt, rep), vrep = g.repeat_kv(vt, rep);
    const int64_t bh = B * heads;
    g.reinterpret_shape(qt, {bh, S, hd});
    g.reinterpret_shape(krep, {bh, S, hd});
    g.reinterpret_shape(vrep, {bh, S, hd});
    const float scale = 1.0f / std::sqrt((float)hd);
    int64_t ctx;
    if (g.no_grad) {
      ctx = g.flash_attention(qt, krep, vrep, scale, causal);
    } else {
      int64_t scores = g.bmm(qt, krep, true);
      int64_t sc = g.alloc_pooled({bh, S, S});
      g.tensors[sc].constant = true;
      ck(eisen_fill_f32(g.stream, (float*)g.tensors[sc].data, scale, bh * S * S), "fill(scale)");
      int64_t scaled = g.mul(scores, sc);
      int64_t masked = scaled;
      if (causal) {
        std::vector<float> md((size_t)S * S, 0.0f);
        for (int64_t r = 0; r < S; ++r)
          for (int64_t c = r + 1; c < S; ++c) md[r * S + c] = -1e20f;
        int64_t mask = g.alloc_pooled({1, S, S});
        g.tensors[mask].constant = true;
        g.load_tensor_data(mask, md.data(), S * S);
        masked = g.add(scaled, mask);
      }
      int64_t probs = g.softmax(masked);
      ctx = g.bmm(probs, vrep, false);
    }
    g.reinterpret_shape(ctx, {B, heads, S, hd});
    int64_t ct = g.transpose_0213(ctx);
    ctx2 = g.reshape(ct, {B, S, hidden});
  }
  if (residual >= 0) {  // residual + out_proj(ctx) in one launch
    const std::vector<int64_t> rs = g.tensors.at(residual).shape;
    int64_t o = g.matmul_add(ctx2, b.o, residual);
    g.reinterpret_shape(o, rs);
    return o;
  }
  return linear_fwd(g, ctx2, b.o);
}

int64_t TransformerLM::block_forward(Graph& g, const BlockParams& b, int64_t x, bool skip_dead_tail,
                                     std::pair<int64_t, int64_t>* kv_out) {
  int64_t n1 = g.rms_norm(x, b.norm1, 1e-5f);
  int64_t r1;
  if (fused) {
    r1 = gqa_forward(g, b, n1, true, x, kv_out);
  } else {
    int64_t at = gqa_forward(g, b, n1, true, -1, kv_out);
    r1 = g.add(x, at);
  }
  int64_t n2 = g.rms_norm(r1, b.norm2, 1e-5f);
  int64_t gd;
  if (fused) {
    gd = g.gate_up_swiglu(n2, b.gate, b.up);  // gate and up projections + SwiGLU in one launch
  } else {
    int64_t go = linear_fwd(g, n2, b.gate);
    int64_t gt = g.silu(go);
    int64_t up = linear_fwd(g, n2, b.up);
    gd = g.mul(gt, up);
  }
  // the down projection's output and the second residual sum feed only the next block: when a
  // checkpointed block is re-run for its backward pass nothing reads them
  FlagGuard skip(g.skip_forward, skip_dead_tail);
  int64_t out;
  if (fused) {
    out = g.matmul_add(gd, b.down, r1);
    g.reinterpret_shape(out, g.tensors[r1].shape);
  } else {
    int64_t f2 = linear_fwd(g, gd, b.down);
    out = g.add(r1, f2);
  }
  return out;
}

int64_t TransformerLM::forward(Graph& g, int64_t x) {
  int64_t h = g.gather(emb, x);
  for (int64_t l = 0; l < layers; ++l) {
    prefetch_block(g, l + 1);
    h = block_forward(g, blocks[(size_t)l], h);
  }
  h = g.rms_norm(h, norm_f, 1e-5f);
  if (tie) return g.matmul_trans_b(h, emb);
  return linear_fwd(g, h, head);
}

int64_t TransformerLM::train_micro_step(Graph& g, int64_t x, const int64_t* targets, int64_t n_targets, bool checkpoint,
                                        const std::function<void(int64_t)>& after_block) {
  std::vector<int32_t> h((size_t)n_targets);
  int64_t valid = 0;
  for (int64_t i = 0; i < n_targets; ++i) {
    if (targets[i] >= vocab) throw EisenException(EISEN_ERR_INVALID, "train_micro_step: target out of range");
    h[i] = targets[i] < 0 ? -1 : (int32_t)targets[i];
    valid += targets[i] >= 0;
  }
  int64_t tid = g.alloc_ids({n_targets}, h.data(), false);
  return train_micro_step_dev(g, x, tid, valid, checkpoint, after_block);
}

int64_t TransformerLM::train_micro_step_dev(Graph& g, int64_t x, int64_t target_ids, int64_t n_valid, bool checkpoint,
                                            const std::function<void(int64_t)>& after_block) {
  if (g.no_grad) throw EisenException(EISEN_ERR_INVALID, "train_micro_step: graph is in no_grad mode");
  const int64_t n_targets = g.tensors.at(target_ids).numel;
  const int64_t tape0 = (int64_t)g.tape.size();
  const bool stash = checkpoint && keep_attention && fused;
  struct StashScope {  // whatever happens, no stashed buffer outlives the step and the mode is off again
    Graph& g;
    ~StashScope() { g.attn_stash_mode = 0; g.attn_stash_slot = -1; g.release_attn_stash(); }
  } stash_scope{g};
  if (stash) g.attn_stash.resize((size_t)layers);
  if (before_block) before_block(-1);
  int64_t h = g.gather(emb, x);
  const int64_t tape_after_emb = (int64_t)g.tape.size();
  std::vector<int64_t> block_in((size_t)layers);
  std::vector<int64_t> block_tape((size_t)layers + 1);
  for (int64_t l = 0; l < layers; ++l) {
    block_in[l] = h;
    block_tape[l] = (int64_t)g.tape.size();
    if (before_block) before_block(l);
    prefetch_block(g, l + 1);  // the next block's streamed weights travel while this block computes
    if (checkpoint) {
      // keep only the block output: run the block without a tape under a save point and move
      // its result into a holder allocated before the save point
      int64_t holder = g.alloc_pooled(g.tensors[h].shape);
      const int64_t sp = g.mark_save_point();
      int64_t r;
      {
        FlagGuard ng(g.no_grad, true);
        g.attn_stash_mode = stash ? 1 : 0;
        g.attn_stash_slot = l;
        r = block_forward(g, blocks[l], h);
        g.attn_stash_mode = 0;
      }
      std::swap(g.tensors[holder].data, g.tensors[r].data);
      g.restore_save_point(sp);
      h = holder;
    } else {
      h = block_forward(g, blocks[l], h);
    }
  }
  block_tape[layers] = (int64_t)g.tape.size();
  if (before_block) before_block(layers);
  int64_t hn = g.rms_norm(h, norm_f, 1e-5f);
  // src/graph/ops/reduction.rs:724-737: mean over the valid rows; all rows masked -> loss 0, no gradient
  const float normalizer = n_valid > 0 ? 1.0f / (float)n_valid : 0.0f;
  int64_t loss;
  if (fused_head) {
    loss = g.lm_head_cross_entropy(hn, tie ? emb : head, target_ids, normalizer, tie, head_chunk_rows);
  } else {
    int64_t logits = tie ? g.matmul_trans_b(hn, emb) : linear_fwd(g, hn, head);
    g.reinterpret_shape(logits, {n_targets, vocab});
    loss = g.ce_device(logits, target_ids, normalizer);
  }

  // ---- backward
  g.seed_grad_ones(loss);
  g.backward_from(block_tape[layers]);  // loss, head, final norm
  if (after_block) after_block(layers);
  if (checkpoint) {
    int64_t out = h;  // holder of the last block's output; its grad is complete now
    for (int64_t l = layers - 1; l >= 0; --l) {
      prefetch_block(g, l - 1);
      const int64_t sp = g.mark_save_point();
      const int64_t t0 = (int64_t)g.tape.size();
      g.attn_stash_mode = stash ? 2 : 0;
      g.attn_stash_slot = l;
      int64_t y = block_forward(g, blocks[l], block_in[l], true);
      g.attn_stash_mode = 0;
      // hand the output gradient to the recomputed output
      HTensor& ty = g.tensors[y];
      HTensor& to = g.tensors[out];
      ty.grad = to.grad;
      ty.grad_dtype = to.grad_dtype;
      ty.grad_init = to.grad_init;
      to.grad = nullptr;
      to.grad_init = false;
      g.backward_from(t0);
      g.tape.resize((size_t)t0);
      g.restore_save_point(sp);
      out = block_in[l];
      if (after_block) after_block(l);
    }
  } else {
    for (int64_t l = layers - 1; l >= 0; --l) {
      for (int64_t i = block_tape[l + 1]; i-- > block_tape[l];) g.tape[i].backward();
      if (after_block) after_block(l);
    }
  }
  for (int64_t i = tape_after_emb; i-- > tape0;) g.tape[i].backward();  // embedding scatter
  if (after_block) after_block(-1);
  return loss;
}

// ------------------------------------------------------------------------------------- generation
namespace {
// logits row `row` of a [rows, vocab] tensor as f32 on the host
void read_logits_row(Graph& g, int64_t logits, int64_t row, int64_t vocab, std::vector<float>& out) {
  const HTensor& t = g.tensors.at(logits);
  out.resize((size_t)vocab);
  if (t.dtype == 0) {
    cuck(cudaMemcpyAsync(out.data(), (const float*)t.data + row * vocab, (size_t)vocab * 4, cudaMemcpyDeviceToHost, g.stream), "D2H(logits)");
  } else {
    float* tmp = static_cast<float*>(g.pool_get((size_t)vocab * 4));
    ck(eisen_cast(g.stream, (const uint16_t*)t.data + row * vocab, 1, tmp, 0, vocab), "cast(logits)");
    cuck(cudaMemcpyAsync(out.data(), tmp, (size_t)vocab * 4, cudaMemcpyDeviceToHost, g.stream), "D2H(logits)");
    g.pool_put(tmp, (size_t)vocab * 4);
  }
  cuck(cudaStreamSynchronize(g.stream), "sync");
  g.check_status();
}
// examples/train_llm.rs:573-578: max_by over partial_cmp keeps the LAST of equal maxima
int32_t argmax_last(const std::vector<float>& v) {
  size_t best = 0;
  for (size_t i = 1; i < v.size(); ++i)
    if (v[i] >= v[best]) best = i;
  return (int32_t)best;
}
}  // namespace

void TransformerLM::generate(Graph& g, const int32_t* prompt, int64_t n_prompt, int64_t max_new, int64_t max_context,
                             bool kv_cache, int32_t* out_tokens, float* last_logits) {
  if (n_prompt <= 0 || max_new <= 0 || max_context <= 0) throw EisenException(EISEN_ERR_INVALID, "generate: needs a prompt, max_new > 0 and max_context > 0");
  for (int64_t i = 0; i < n_prompt; ++i)
    if (prompt[i] < 0 || prompt[i] >= vocab) throw EisenException(EISEN_ERR_INVALID, "generate: prompt token outside [0, vocab)");
  FlagGuard ng(g.no_grad, true);
  std::vector<float> row;
  if (!kv_cache) {
    // the reference's loop: the whole (windowed) context goes through forward() for every token
    std::vector<int32_t> tokens(prompt, prompt + n_prompt);
    for (int64_t i = 0; i < max_new; ++i) {
      const int64_t start = std::max<int64_t>(0, (int64_t)tokens.size() - max_context);
      const int64_t csl = (int64_t)tokens.size() - start;
      int64_t x = g.alloc_ids({1, csl}, tokens.data() + start, false);
      int64_t logits = forward(g, x);
      read_logits_row(g, logits, csl - 1, vocab, row);
      const int32_t next = argmax_last(row);
      out_tokens[i] = next;
      tokens.push_back(next);
      g.clear_activations();
    }
    if (last_logits) std::memcpy(last_logits, row.data(), (size_t)vocab * 4);
    return;
  }
  const int64_t max_len = n_prompt + max_new;
  if (max_len > max_context)
    throw EisenException(EISEN_ERR_LIMIT, "generate: with a KV cache prompt + new tokens must fit max_context "
                                          "(a sliding window re-positions every cached key); use kv_cache = 0");
  const int64_t hd = hidden / heads, kvd = kv_heads * hd;
  const int dt = g.act_dtype();
  const size_t esz = dt == 1 ? 2 : 4;
  const size_t cache_bytes = (size_t)max_len * kvd * esz;
  std::vector<char*> kc((size_t)layers), vc((size_t)layers);
  struct Release {
    Graph& g; std::vector<char*>&a, &b; size_t bytes;
    ~Release() { for (char* p : a) g.pool_put(p, bytes); for (char* p : b) g.pool_put(p, bytes); }
  } release{g, kc, vc, cache_bytes};
  for (int64_t l = 0; l < layers; ++l) { kc[l] = nullptr; vc[l] = nullptr; }
  for (int64_t l = 0; l < layers; ++l) {
    kc[l] = static_cast<char*>(g.pool_get(cache_bytes));
    vc[l] = static_cast<char*>(g.pool_get(cache_bytes));
  }
  const float* tab = g.rope_table(max_len, hd);
  const float scale = 1.0f / std::sqrt((float)hd);
  // ---- the prompt in one pass; every layer's rotated keys and its values go to the cache
  {
    int64_t x = g.alloc_ids({1, n_prompt}, prompt, false);
    int64_t h = g.gather(emb, x);
    for (int64_t l = 0; l < layers; ++l) {
      std::pair<int64_t, int64_t> kv;
      h = block_forward(g, blocks[l], h, false, &kv);
      cuck(cudaMemcpyAsync(kc[l], g.tensors[kv.first].data, (size_t)n_prompt * kvd * esz, cudaMemcpyDeviceToDevice, g.stream), "copy(k cache)");
      cuck(cudaMemcpyAsync(vc[l], g.tensors[kv.second].data, (size_t)n_prompt * kvd * esz, cudaMemcpyDeviceToDevice, g.stream), "copy(v cache)");
    }
    h = g.rms_norm(h, norm_f, 1e-5f);
    int64_t logits = tie ? g.matmul_trans_b(h, emb) : linear_fwd(g, h, head);
    read_logits_row(g, logits, n_prompt - 1, vocab, row);
    out_tokens[0] = argmax_last(row);
    g.clear_activations();
  }
  // ---- one row per further token
  for (int64_t i = 1; i < max_new; ++i) {
    const int64_t pos = n_prompt + i - 1;  // position of the token fed in
    const int32_t tok = out_tokens[i - 1];
    int64_t x = g.alloc_ids({1, 1}, &tok, false);
    int64_t h = g.gather(emb, x);
    const float* tab_pos = tab + pos * (hd / 2) * 2;
    for (int64_t l = 0; l < layers; ++l) {
      const BlockParams& b = blocks[l];
      int64_t n1 = g.rms_norm(h, b.norm1, 1e-5f);
      int64_t q = g.matmul(n1, b.q), k = g.matmul(n1, b.k), v = g.matmul(n1, b.v);
      int64_t qr = g.alloc_pooled({1, hidden});
      ck(eisen_rope(g.stream, g.tensors[q].data, g.tensors[qr].data, tab_pos, 1, 1, hidden, hd, dt, 0, 0), "rope(q)");
      ck(eisen_rope(g.stream, g.tensors[k].data, kc[l] + (size_t)pos * kvd * esz, tab_pos, 1, 1, kvd, hd, dt, 0, 0), "rope(k)");
      ck(eisen_cast(g.stream, g.tensors[v].data, dt, vc[l] + (size_t)pos * kvd * esz, dt, kvd), "copy(v)");
      int64_t ctx = g.alloc_pooled({1, hidden});
      ck(eisen_attn_decode(g.stream, g.tensors[qr].data, kc[l], vc[l], g.tensors[ctx].data, pos + 1, heads, kv_heads, hd, kvd,
                           scale, dt),
         "attn_decode");
      int64_t r1 = g.add(h, g.matmul(ctx, b.o));
      int64_t n2 = g.rms_norm(r1, b.norm2, 1e-5f);
      int64_t go = g.matmul(n2, b.gate), up = g.matmul(n2, b.up);
      int64_t gd = fused ? g.swiglu(go, up) : g.mul(g.silu(go), up);
      h = g.add(r1, g.matmul(gd, b.down));
    }
    h = g.rms_norm(h, norm_f, 1e-5f);
    int64_t logits = tie ? g.matmul_trans_b(h, emb) : g.matmul(h, head);
    read_logits_row(g, logits, 0, vocab, row);
    out_tokens[i] = argmax_last(row);
    g.clear_activations();
  }
  if (last_logits) std::memcpy(last_logits, row.data(), (size_t)vocab * 4);
}

// ------------------------------------------------------------------------------------- AdamW
AdamW::AdamW(Graph& g_, std::vector<int64_t> params_, float lr_) : lr(lr_), g(g_), params(std::move(params_)) {
  // one launch over the arena when the parameter list is exactly the arena's content
  int64_t in_arena = 0, arena_elems = 0;
  for (int64_t p : params) {
    const HTensor& t = g.tensors.at(p);
    if (g.arena_w && t.data >= (void*)g.arena_w && t.data < (void*)(g.arena_w + g.arena_cap)) {
      ++in_arena;
      arena_elems += (t.numel + 63) / 64 * 64;
    }
  }
  flat = g.arena_w && in_arena == (int64_t)params.size() && arena_elems == g.arena_used;
  if (flat) {
    total = g.arena_used;
  } else {
    for (int64_t p : params) {
      offsets.push_back(total);
      if (!g.tensors.at(p).host_homed) total += (g.tensors.at(p).numel + 63) / 64 * 64;
    }
  }
  const size_t bytes = (size_t)std::max<int64_t>(total, 64) * 4;
  cuck(cudaMalloc(&m, bytes), "cudaMalloc(adam m)");
  cuck(cudaMalloc(&v, bytes), "cudaMalloc(adam v)");
  cuck(cudaMemsetAsync(m, 0, bytes, g.stream), "memset");
  cuck(cudaMemsetAsync(v, 0, bytes, g.stream), "memset");
  if (!flat) {
    for (size_t i = 0; i < params.size(); ++i) {
      const HTensor& tt = g.tensors[params[i]];
      if (!tt.host_homed) {
        m_ptr.push_back(m + offsets[i]);
        v_ptr.push_back(v + offsets[i]);
        continue;
      }
      for (std::vector<float*>* dst : {&m_ptr, &v_ptr}) {
        void* hp = nullptr;
        const size_t hb = (size_t)std::max<int64_t>(tt.numel, 4) * 4;
        cuck(cudaHostAlloc(&hp, hb, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc(adam moments)");
        std::memset(hp, 0, hb);
        host_moments.push_back((float*)hp);
        dst->push_back((float*)hp);
      }
    }
  }
  int64_t longest = 64;
  for (int64_t p : params) longest = std::max(longest, g.tensors[p].numel);
  cuck(cudaMalloc(&sumsq_dev, 64), "cudaMalloc(sumsq)");
  cuck(cudaMalloc(&sumsq_ws, (size_t)eisen_sumsq_workspace_bytes(std::max<int64_t>(std::max(total, longest), 64))), "cudaMalloc(sumsq ws)");
  g.device_bytes_allocated += 2 * bytes;
}

AdamW::AdamW(Graph& g_, std::vector<int64_t> params_, float lr_, std::vector<std::pair<int64_t, int64_t>> pieces_)
    : lr(lr_), g(g_), params(std::move(params_)), pieces(std::move(pieces_)) {
  if (!g.arena_w) throw EisenException(EISEN_ERR_INVALID, "sharded AdamW needs the flat parameter arena");
  for (int64_t p : params) {
    const HTensor& t = g.tensors.at(p);
    if (!(t.data >= (void*)g.arena_w && t.data < (void*)(g.arena_w + g.arena_cap)))
      throw EisenException(EISEN_ERR_INVALID, "sharded AdamW: every parameter must live in the arena");
  }
  flat = true;
  total = g.arena_used;
  int64_t mine = 0;
  for (auto& pc : pieces) {
    if (pc.first < 0 || pc.second < pc.first || pc.second > total || (pc.first % 4) || (pc.second % 4))
      throw EisenException(EISEN_ERR_INVALID, "sharded AdamW: a piece must be a 4-element-aligned range inside the arena");
    piece_state_off.push_back(mine);
    mine += pc.second - pc.first;
  }
  const size_t bytes = (size_t)std::max<int64_t>(mine, 64) * 4;
  cuck(cudaMalloc(&m, bytes), "cudaMalloc(adam m)");
  cuck(cudaMalloc(&v, bytes), "cudaMalloc(adam v)");
  cuck(cudaMemsetAsync(m, 0, bytes, g.stream), "memset");
  cuck(cudaMemsetAsync(v, 0, bytes, g.stream), "memset");
  cuck(cudaMalloc(&sumsq_dev, 64), "cudaMalloc(sumsq)");
  cuck(cudaMemsetAsync(sumsq_dev, 0, 64, g.stream), "memset");
  cuck(cudaMalloc(&sumsq_ws, (size_t)eisen_sumsq_workspace_bytes(std::max<int64_t>(total, 64))), "cudaMalloc(sumsq ws)");
  g.device_bytes_allocated += 2 * bytes;
}

void AdamW::sumsq_piece(size_t i, bool accumulate, cudaStream_t s) {
  const auto& pc = pieces.at(i);
  if (pc.second == pc.first) {
    if (!accumulate) cuck(cudaMemsetAsync(sumsq_dev, 0, 8, s), "memset(sumsq)");
    return;
  }
  ck(eisen_sumsq(s, g.arena_g + pc.first, pc.second - pc.first, sumsq_ws, sumsq_dev, accumulate ? 1 : 0), "sumsq(piece)");
}

void AdamW::step_piece(size_t i, float max_norm, float grad_scale, cudaStream_t s, bool zero_grads) {
  const auto& pc = pieces.at(i);
  if (pc.second == pc.first) return;
  float p1 = 1.0f, p2 = 1.0f;
  for (int64_t k = 0; k < t; ++k) { p1 *= beta1; p2 *= beta2; }
  const float bc1 = 1.0f / (1.0f - p1), bc2 = 1.0f / (1.0f - p2);
  const int64_t so = piece_state_off[i];
  void* shadow = g.arena_shadow ? (void*)((uint16_t*)g.arena_shadow + pc.first) : nullptr;
  ck(eisen_adamw_step_ex(s ? s : g.stream, g.arena_w + pc.first, shadow, g.arena_g + pc.first, m + so, v + so,
                         pc.second - pc.first, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale,
                         max_norm > 0.0f ? sumsq_dev : nullptr, max_norm, nullptr, zero_grads ? 1 : 0),
     "adamw_step(piece)");
}

int64_t AdamW::state_elems() const {
  int64_t n = 0;
  if (!pieces.empty()) {
    for (const auto& pc : pieces) n += pc.second - pc.first;
    return n;
  }
  if (flat) return total;
  for (int64_t p : params) n += g.tensors[p].numel;
  return n;
}

namespace {
struct MomentSegment { float* m; float* v; int64_t n; };
}
static std::vector<MomentSegment> moment_segments(const AdamW& o) {
  std::vector<MomentSegment> segs;
  if (!o.pieces.empty() || o.flat) {
    segs.push_back({o.m, o.v, o.state_elems()});
  } else {
    for (size_t i = 0; i < o.params.size(); ++i) segs.push_back({o.m_ptr[i], o.v_ptr[i], o.g.tensors[o.params[i]].numel});
  }
  return segs;
}

namespace {
struct OptStateHeader {
  char magic[8];          // "EISENOPT"
  int64_t version;        // 1
  int64_t t;              // optimizer steps taken
  int64_t elems;          // f32 elements of m (and of v) that follow
  int64_t total;          // elements the optimizer covers across all ranks
  int64_t n_pieces;       // 0: one contiguous state; else the [lo, hi) ranges follow the header
  float lr, beta1, beta2, eps, weight_decay;
  float reserved[3];
};
}  // namespace

void AdamW::save_state(const char* path) {
  cuck(cudaStreamSynchronize(g.stream), "sync");
  FILE* f = fopen(path, "wb");
  if (!f) throw EisenException(EISEN_ERR_INVALID, std::string("optimizer save_state: cannot create ") + path);
  OptStateHeader h{};
  std::memcpy(h.magic, "EISENOPT", 8);
  h.version = 1; h.t = t; h.elems = state_elems(); h.total = total; h.n_pieces = (int64_t)pieces.size();
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = weight_decay;
  bool ok = fwrite(&h, sizeof(h), 1, f) == 1;
  for (const auto& pc : pieces) {
    const int64_t r[2] = {pc.first, pc.second};
    ok = ok && fwrite(r, sizeof(r), 1, f) == 1;
  }
  std::vector<float> buf((size_t)std::max<int64_t>(std::min<int64_t>(h.elems, 1 << 24), 1));
  const std::vector<MomentSegment> segs = moment_segments(*this);
  for (int which = 0; which < 2; ++which) {
    for (const MomentSegment& sg : segs) {
      const float* src = which ? sg.v : sg.m;
      for (int64_t off = 0; off < sg.n && ok; off += (int64_t)buf.size()) {
        const size_t n = (size_t)std::min<int64_t>((int64_t)buf.size(), sg.n - off);
        cuck(cudaMemcpy(buf.data(), src + off, n * 4, cudaMemcpyDefault), "D2H(optimizer state)");
        ok = fwrite(buf.data(), 4, n, f) == n;
      }
    }
  }
  ok = (fclose(f) == 0) && ok;
  if (!ok) throw EisenException(EISEN_ERR_INVALID, "optimizer save_state: short write");
}

void AdamW::load_state(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) throw EisenException(EISEN_ERR_INVALID, std::string("optimizer load_state: cannot open ") + path);
  struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{f};
  OptStateHeader h{};
  if (fread(&h, sizeof(h), 1, f) != 1 || std::memcmp(h.magic, "EISENOPT", 8) != 0 || h.version != 1)
    throw EisenException(EISEN_ERR_INVALID, "optimizer load_state: not an optimizer state file of this library");
  if (h.elems != state_elems() || h.total != total || h.n_pieces != (int64_t)pieces.size())
    throw EisenException(EISEN_ERR_INVALID, "optimizer load_state: the file was written for another model or another sharding");
  for (const auto& pc : pieces) {
    int64_t r[2];
    if (fread(r, sizeof(r), 1, f) != 1 || r[0] != pc.first || r[1] != pc.second)
      throw EisenException(EISEN_ERR_INVALID, "optimizer load_state: the file's ranges differ from this rank's");
  }
  cuck(cudaStreamSynchronize(g.stream), "sync");
  std::vector<float> buf((size_t)std::max<int64_t>(std::min<int64_t>(h.elems, 1 << 24), 1));
  const std::vector<MomentSegment> segs = moment_segments(*this);
  for (int which = 0; which < 2; ++which) {
    for (const MomentSegment& sg : segs) {
      float* dst = which ? sg.v : sg.m;
      for (int64_t off = 0; off < sg.n; off += (int64_t)buf.size()) {
        const size_t n = (size_t)std::min<int64_t>((int64_t)buf.size(), sg.n - off);
        if (fread(buf.data(), 4, n, f) != n) throw EisenException(EISEN_ERR_INVALID, "optimizer load_state: short read");
        cuck(cudaMemcpy(dst + off, buf.data(), n * 4, cudaMemcpyDefault), "H2D(optimizer state)");
      }
    }
  }
  t = h.t;
  lr = h.lr; beta1 = h.beta1; beta2 = h.beta2; eps = h.eps; weight_decay = h.weight_decay;
}

AdamW::~AdamW() {
  cudaStreamSynchronize(g.stream);
  cudaFree(m);
  cudaFree(v);
  cudaFree(sumsq_dev);
  cudaFree(sumsq_ws);
  for (float* p : host_moments) cudaFreeHost(p);
  if (hyper_host) cudaFreeHost(hyper_host);
  if (hyper_dev) cudaFree(hyper_dev);
}

void AdamW::zero_grad() {
  if (flat) {
    cuck(cudaMemsetAsync(g.arena_g, 0, (size_t)total * 4, g.stream), "memset(grads)");
    return;
  }
  for (int64_t p : params) g.zero_grad(p);
}

// squared norm of all parameter gradients into sumsq_dev (f64, device)
static void grad_sumsq(AdamW& o) {
  Graph& g = o.g;
  if (o.flat) {
    ck(eisen_sumsq(g.stream, g.arena_g, o.total, o.sumsq_ws, o.sumsq_dev, 0), "sumsq");
    return;
  }
  bool first = true;
  for (int64_t p : o.params) {
    const HTensor& t = g.tensors[p];
    ck(eisen_sumsq(g.stream, (const float*)t.grad, t.numel, o.sumsq_ws, o.sumsq_dev, first ? 0 : 1), "sumsq");
    first = false;
  }
}

float AdamW::clip_grad_norm(float max_norm, float* coef_out) {
  grad_sumsq(*this);
  double ss = 0.0;
  cuck(cudaMemcpyAsync(&ss, sumsq_dev, 8, cudaMemcpyDeviceToHost, g.stream), "D2H(sumsq)");
  cuck(cudaStreamSynchronize(g.stream), "sync");
  const float norm = (float)std::sqrt(ss);
  const float coef = norm > 0.0f ? std::min(max_norm / (norm + 1e-6f), 1.0f) : 1.0f;
  if (coef < 1.0f) {
    if (flat) {
      ck(eisen_scale_f32(g.stream, g.arena_g, coef, total), "scale");
    } else {
      for (int64_t p : params) ck(eisen_scale_f32(g.stream, (float*)g.tensors[p].grad, coef, g.tensors[p].numel), "scale");
    }
  }
  if (coef_out) *coef_out = coef;
  return norm;
}

// t += 1 and the step's scalars into the page-locked record a captured step copies from
void AdamW::advance() {
  if (!hyper_host) {
    cuck(cudaHostAlloc((void**)&hyper_host, 16, cudaHostAllocDefault), "cudaHostAlloc(adam scalars)");
    cuck(cudaMalloc((void**)&hyper_dev, 16), "cudaMalloc(adam scalars)");
  }
  t += 1;
  float p1 = 1.0f, p2 = 1.0f;
  for (int64_t i = 0; i < t; ++i) { p1 *= beta1; p2 *= beta2; }
  hyper_host[0] = lr;
  hyper_host[1] = 1.0f / (1.0f - p1);
  hyper_host[2] = 1.0f / (1.0f - p2);
  hyper_host[3] = 0.0f;
}

void AdamW::launch(float grad_scale, const double* sumsq, float max_norm) {
  const float* hyper = nullptr;
  if (g.capturing) {
    // recorded once, replayed every step: the scalars come from device memory (see advance())
    if (!hyper_host) throw EisenException(EISEN_ERR_INVALID, "optimizer step inside a capture: call eisen_optim_advance first");
    cuck(cudaMemcpyAsync(hyper_dev, hyper_host, 16, cudaMemcpyHostToDevice, g.stream), "H2D(adam scalars)");
    hyper = hyper_dev;
  } else {
    t += 1;
  }
  // src/nn/optim.rs:336-338: reciprocal bias corrections from powi
  float p1 = 1.0f, p2 = 1.0f;
  for (int64_t i = 0; i < t; ++i) { p1 *= beta1; p2 *= beta2; }
  const float bc1 = 1.0f / (1.0f - p1), bc2 = 1.0f / (1.0f - p2);
  if (flat) {
    ck(eisen_adamw_step_dev(g.stream, g.arena_w, g.arena_shadow, g.arena_g, m, v, total, lr, beta1, beta2, eps, weight_decay,
                            bc1, bc2, grad_scale, sumsq, max_norm, hyper),
       "adamw_step");
    return;
  }
  for (size_t i = 0; i < params.size(); ++i) {
    HTensor& tt = g.tensors[params[i]];
    ck(eisen_adamw_step_dev(g.stream, (float*)tt.data, tt.shadow, (const float*)tt.grad, m_ptr[i], v_ptr[i],
                            tt.numel, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, sumsq, max_norm, hyper),
       "adamw_step");
  }
  g.invalidate_staged_weights();  // staged copies of host-homed weights are stale now
}

void AdamW::step() { launch(1.0f, nullptr, 0.0f); }

void AdamW::step_fused(float max_norm, float grad_scale) {
  if (max_norm > 0.0f) {
    grad_sumsq(*this);
    launch(grad_scale, sumsq_dev, max_norm);
  } else {
    launch(grad_scale, nullptr, 0.0f);
  }
}

}  // namespace eisen
