// Hugging Face export of a trained TransformerLM: `model.safetensors` + `config.json`.
//
// Follows the reference's exporter (examples/export_hf_pipeline.rs:34-55, 200-300 and
// src/tools/huggingface.rs:88-146):
//   * tensor names of LlamaForCausalLM, in the order embedding, per layer (input_layernorm, q, k, v, o,
//     post_attention_layernorm, gate, up, down), final norm, lm_head (left out when tied);
//   * Linear weights are stored [in, out] here and [out, in] there: every 2-D tensor except the
//     embedding is transposed;
//   * the engine rotates interleaved pairs (2p, 2p + 1) of a head, Hugging Face rotates (p, p + D/2):
//     the rows of the transposed q and k weights are permuted accordingly, per head;
//   * safetensors layout: u64 header length, JSON header (entries sorted by name, padded with spaces
//     to a multiple of 8 bytes), f32 little-endian payload in the tensor order above;
//   * config.json with the keys of the pipeline, num_key_value_heads = the number of KV heads
//     (src/tools/huggingface.rs:70-71 writes num_attention_heads there; the pipeline's value is the
//     right one for a GQA model).
// The f32 master weights are written (the reference keeps bf16 parameters in bf16 mode and exports
// their f32 widening).
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "../../../include/eisen_b200.h"
#include "../errors.h"
#include "graph.h"

namespace eisen {

namespace {

std::vector<float> transpose_2d(const std::vector<float>& d, int64_t rows, int64_t cols) {  // pipeline :24-32
  std::vector<float> t(d.size());
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) t[(size_t)(c * rows + r)] = d[(size_t)(r * cols + c)];
  return t;
}

// rows [h*D + 2p, h*D + 2p + 1] -> rows [h*D + p, h*D + D/2 + p] of an [out, in] matrix (pipeline :34-55)
std::vector<float> permute_rope_hf(const std::vector<float>& d, int64_t heads, int64_t head_dim, int64_t in_features) {
  std::vector<float> o(d.size(), 0.0f);
  for (int64_t h = 0; h < heads; ++h)
    for (int64_t p = 0; p < head_dim / 2; ++p) {
      const int64_t src1 = h * head_dim + 2 * p, src2 = src1 + 1;
      const int64_t dst1 = h * head_dim + p, dst2 = h * head_dim + head_dim / 2 + p;
      std::copy(d.begin() + src1 * in_features, d.begin() + (src1 + 1) * in_features, o.begin() + dst1 * in_features);
      std::copy(d.begin() + src2 * in_features, d.begin() + (src2 + 1) * in_features, o.begin() + dst2 * in_features);
    }
  return o;
}

struct Entry {
  std::vector<int64_t> shape;
  size_t begin, end;
};

}  // namespace

void export_hf(Graph& g, const TransformerLM& lm, const char* safetensors_path, const char* config_path,
               int64_t max_position_embeddings) {
  g.synchronize();
  const int64_t hd = lm.hidden / lm.heads;
  std::vector<std::pair<std::string, Entry>> order;
  std::vector<float> payload;
  auto add = [&](const std::string& name, int64_t id, bool transpose, int64_t rope_heads) {
    const HTensor& t = g.tensors.at(id);
    std::vector<float> data((size_t)t.numel);
    g.sync_to_cpu(id, data.data());
    std::vector<int64_t> shape = t.shape;
    if (transpose) {
      data = transpose_2d(data, shape[0], shape[1]);
      std::swap(shape[0], shape[1]);
    }
    if (rope_heads > 0) data = permute_rope_hf(data, rope_heads, hd, shape[1]);
    Entry e{shape, payload.size() * 4, 0};
    payload.insert(payload.end(), data.begin(), data.end());
    e.end = payload.size() * 4;
    order.emplace_back(name, e);
  };
  add("model.embed_tokens.weight", lm.emb, false, 0);
  for (int64_t i = 0; i < lm.layers; ++i) {
    const BlockParams& b = lm.blocks[(size_t)i];
    const std::string p = "model.layers." + std::to_string(i) + ".";
    add(p + "input_layernorm.weight", b.norm1, false, 0);
    add(p + "self_attn.q_proj.weight", b.q, true, lm.heads);
    add(p + "self_attn.k_proj.weight", b.k, true, lm.kv_heads);
    add(p + "self_attn.v_proj.weight", b.v, true, 0);
    add(p + "self_attn.o_proj.weight", b.o, true, 0);
    add(p + "post_attention_layernorm.weight", b.norm2, false, 0);
    add(p + "mlp.gate_proj.weight", b.gate, true, 0);
    add(p + "mlp.up_proj.weight", b.up, true, 0);
    add(p + "mlp.down_proj.weight", b.down, true, 0);
  }
  add("model.norm.weight", lm.norm_f, false, 0);
  if (!lm.tie) add("lm_head.weight", lm.head, true, 0);

  std::map<std::string, Entry> sorted(order.begin(), order.end());  // BTreeMap order of the reference
  std::string header = "{";
  bool first = true;
  for (const auto& kv : sorted) {
    if (!first) header += ",";
    first = false;
    header += "\"" + kv.first + "\":{\"dtype\":\"F32\",\"shape\":[";
    for (size_t i = 0; i < kv.second.shape.size(); ++i) header += (i ? "," : "") + std::to_string(kv.second.shape[i]);
    header += "],\"data_offsets\":[" + std::to_string(kv.second.begin) + "," + std::to_string(kv.second.end) + "]}";
  }
  header += "}";
  while (header.size() % 8) header += ' ';

  FILE* f = fopen(safetensors_path, "wb");
  if (!f) throw EisenException(EISEN_ERR_INVALID, std::string("export_hf: cannot create ") + safetensors_path);
  const uint64_t hl = header.size();
  bool ok = fwrite(&hl, 8, 1, f) == 1 && fwrite(header.data(), 1, header.size(), f) == header.size() &&
            fwrite(payload.data(), 4, payload.size(), f) == payload.size();
  ok = (fclose(f) == 0) && ok;
  if (!ok) throw EisenException(EISEN_ERR_INVALID, "export_hf: short write to the safetensors file");

  if (config_path) {
    FILE* c = fopen(config_path, "w");
    if (!c) throw EisenException(EISEN_ERR_INVALID, std::string("export_hf: cannot create ") + config_path);
    fprintf(c,
            "{\n  \"architectures\": [\"LlamaForCausalLM\"],\n  \"model_type\": \"llama\",\n  \"vocab_size\": %lld,\n"
            "  \"hidden_size\": %lld,\n  \"intermediate_size\": %lld,\n  \"num_hidden_layers\": %lld,\n"
            "  \"num_attention_heads\": %lld,\n  \"num_key_value_heads\": %lld,\n  \"max_position_embeddings\": %lld,\n"
            "  \"rms_norm_eps\": 1e-05,\n  \"rope_theta\": 10000.0,\n  \"bos_token_id\": 1,\n  \"eos_token_id\": 2,\n"
            "  \"pad_token_id\": 0,\n  \"hidden_act\": \"silu\",\n  \"tie_word_embeddings\": %s,\n"
            "  \"initializer_range\": 0.02,\n  \"torch_dtype\": \"float32\"\n}\n",
            (long long)lm.vocab, (long long)lm.hidden, (long long)lm.ffn, (long long)lm.layers, (long long)lm.heads,
            (long long)lm.kv_heads, (long long)max_position_embeddings, lm.tie ? "true" : "false");
    fclose(c);
  }
}

// Weights-only checkpoint of examples/train_llm.rs:92-105 (`save_weights`): every parameter tensor in id
// order, f32 little-endian, nothing else; the file the reference's converter
// (examples/export_hf_pipeline.rs:187-196) reads.  Id tensors that sit below the parameter watermark
// are not parameters and are skipped.
void save_weights(Graph& g, const char* path) {
  g.synchronize();
  FILE* f = fopen(path, "wb");
  if (!f) throw EisenException(EISEN_ERR_INVALID, std::string("save_weights: cannot create ") + path);
  std::vector<float> buf;
  bool ok = true;
  for (int64_t i = 0; i < g.num_params && ok; ++i) {
    const HTensor& t = g.tensors[(size_t)i];
    if (t.dtype == DT_I32) continue;
    buf.resize((size_t)t.numel);
    g.sync_to_cpu(i, buf.data());
    ok = fwrite(buf.data(), 4, buf.size(), f) == buf.size();
  }
  ok = (fclose(f) == 0) && ok;
  if (!ok) throw EisenException(EISEN_ERR_INVALID, "save_weights: short write");
}

// The inverse (the reference has none): fills the parameters of an identically built model from such a
// file; in Bf16Mixed mode the bf16 copies are refreshed too.  The file size must match exactly.
void load_weights(Graph& g, const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) throw EisenException(EISEN_ERR_INVALID, std::string("load_weights: cannot open ") + path);
  fseek(f, 0, SEEK_END);
  const long long bytes = ftell(f);
  fseek(f, 0, SEEK_SET);
  long long want = 0;
  for (int64_t i = 0; i < g.num_params; ++i)
    if (g.tensors[(size_t)i].dtype != DT_I32) want += g.tensors[(size_t)i].numel * 4;
  if (bytes != want) {
    fclose(f);
    throw EisenException(EISEN_ERR_INVALID, "load_weights: the file does not hold exactly this model's parameters");
  }
  std::vector<float> buf;
  for (int64_t i = 0; i < g.num_params; ++i) {
    const HTensor& t = g.tensors[(size_t)i];
    if (t.dtype == DT_I32) continue;
    buf.resize((size_t)t.numel);
    if (fread(buf.data(), 4, buf.size(), f) != buf.size()) {
      fclose(f);
      throw EisenException(EISEN_ERR_INVALID, "load_weights: short read");
    }
    g.load_tensor_data(i, buf.data(), t.numel);
  }
  fclose(f);
  g.synchronize();
}

}  // namespace eisen
