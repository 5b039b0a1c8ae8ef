// Input side of the training step: pre-tokenised u16 token files -> int32 id / target batches.
//
// Follows BinaryDataLoader (src/data/dataloader.rs:89-214) and the fill-in-the-middle transform
// (src/data/fim.rs:96-180) of the reference:
//   * the file is a flat little-endian u16 token stream; a batch consumes batch * (seq_len + 1)
//     consecutive tokens, sequence b starting at b * (seq_len + 1); x = tokens [0, seq_len),
//     y = tokens [1, seq_len + 1); a trailing partial batch is dropped;
//   * one xorshift64 draw per sequence decides whether it is FIM-transformed (the draw is made
//     even when FIM is off, dataloader.rs:162); the split points and the PSM / SPM choice come from
//     the same generator through the sampling rules of the `rand` crate the reference pins
//     (rand 0.8.5: widening-multiply rejection for integer ranges, top 24 bits for f32);
//   * targets of positions outside the middle span are the ignore index.
// Differences on purpose: ids are int32 (the reference hands x out as f32 and targets as usize) and
// the ignore index is -1 (usize::MAX there), the values the device-side cross entropy takes.
//
// The loader writes into caller-provided host buffers (pinned ones when they are to be copied to
// the device asynchronously); it allocates no device memory and touches no CUDA API.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../../include/eisen_b200.h"
#include "../errors.h"

namespace {

using eisen::set_error;

struct XorShift64 {  // dataloader.rs:201-207, 214-221
  uint64_t s;
  uint64_t next_u64() {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    return s;
  }
  uint32_t next_u32() { return (uint32_t)next_u64(); }
  // dataloader.rs:201-207: (state >> 11) as f32 / 2^53 as f32
  float unit_f32() { return (float)(next_u64() >> 11) / (float)(1ull << 53); }
  // rand 0.8.5, Standard for f32: 24 random bits scaled by 2^-24
  float gen_f32() { return (float)(next_u32() >> 8) * (1.0f / 16777216.0f); }
  // rand 0.8.5, UniformInt<usize>::sample_single on a 64-bit target, range [low, high)
  uint64_t gen_range(uint64_t low, uint64_t high) {
    const uint64_t range = high - low;  // high > low is the caller's business (as in the crate)
    if (range == 0) return low + next_u64();
    int lz = 0;
    for (uint64_t r = range; !(r >> 63); r <<= 1) ++lz;
    const uint64_t zone = (range << lz) - 1;
    for (;;) {
      const unsigned __int128 m = (unsigned __int128)next_u64() * (unsigned __int128)range;
      const uint64_t hi = (uint64_t)(m >> 64), lo = (uint64_t)m;
      if (lo <= zone) return low + hi;
    }
  }
};

struct Loader {
  FILE* f = nullptr;
  long long seq_len = 0, batch = 0, total_batches = 0;
  std::vector<int32_t> buffer;  // tokens read from the file and not yet consumed
  size_t head = 0;              // first unconsumed token of `buffer`
  bool fim = false;
  long long fim_prefix = 0, fim_suffix = 0, fim_middle = 0, fim_pad = 0;
  float fim_rate = 0.5f, spm_rate = 0.5f;
  XorShift64 rng{1337};
  ~Loader() { if (f) fclose(f); }
};

constexpr int32_t IGNORE = -1;

// src/data/fim.rs:96-168; out_x / out_mask have seq_len entries
void apply_fim(const int32_t* tok, long long n, const Loader& L, XorShift64& rng, int32_t* out_x, uint8_t* out_mask) {
  const long long seq_len = L.seq_len;
  if (n < 4) {  // fim.rs:105-109: padded copy, everything trained
    for (long long i = 0; i < seq_len; ++i) {
      out_x[i] = i < n ? tok[i] : (int32_t)L.fim_pad;
      out_mask[i] = 1;
    }
    return;
  }
  const long long lo = (long long)rng.gen_range(1, (uint64_t)(n - 2));
  const long long hi = (long long)rng.gen_range((uint64_t)(lo + 1), (uint64_t)(n - 1));
  const bool use_spm = rng.gen_f32() < L.spm_rate;
  long long w = 0;
  auto push = [&](int32_t t, uint8_t m) {
    if (w < seq_len) { out_x[w] = t; out_mask[w] = m; }
    ++w;
  };
  auto push_slice = [&](long long a, long long b, uint8_t m) { for (long long i = a; i < b; ++i) push(tok[i], m); };
  if (use_spm) {  // <fim_suffix> suffix <fim_prefix> prefix <fim_middle> middle
    push((int32_t)L.fim_suffix, 0); push_slice(hi, n, 0);
    push((int32_t)L.fim_prefix, 0); push_slice(0, lo, 0);
  } else {        // <fim_prefix> prefix <fim_suffix> suffix <fim_middle> middle
    push((int32_t)L.fim_prefix, 0); push_slice(0, lo, 0);
    push((int32_t)L.fim_suffix, 0); push_slice(hi, n, 0);
  }
  push((int32_t)L.fim_middle, 0);
  push_slice(lo, hi, 1);
  for (; w < seq_len; ++w) { out_x[w] = (int32_t)L.fim_pad; out_mask[w] = 0; }
}

Loader* H(void* h) { return static_cast<Loader*>(h); }

}  // namespace

extern "C" {

int eisen_loader_open(const char* path, long long seq_len, long long batch, void** handle_out) {
  if (!path || !handle_out || seq_len <= 0 || batch <= 0) { set_error("loader_open: bad argument"); return EISEN_ERR_INVALID; }
  std::unique_ptr<Loader> L(new Loader());
  L->f = fopen(path, "rb");
  if (!L->f) { set_error((std::string("loader_open: cannot open ") + path).c_str()); return EISEN_ERR_INVALID; }
  fseek(L->f, 0, SEEK_END);
  const long long bytes = ftell(L->f);
  fseek(L->f, 0, SEEK_SET);
  L->seq_len = seq_len;
  L->batch = batch;
  L->total_batches = (bytes / 2) / (batch * (seq_len + 1));  // dataloader.rs:105-108
  *handle_out = L.release();
  return 0;
}

int eisen_loader_close(void* h) {
  delete H(h);
  return 0;
}

long long eisen_loader_total_batches(void* h) { return h ? H(h)->total_batches : 0; }

// FIM tokens are base_vocab .. base_vocab + 3 = prefix, suffix, middle, pad (fim.rs:36-44)
int eisen_loader_set_fim(void* h, long long base_vocab, float rate, float spm_rate) {
  if (!h || base_vocab < 0) { set_error("loader_set_fim: bad argument"); return EISEN_ERR_INVALID; }
  Loader& L = *H(h);
  L.fim = true;
  L.fim_prefix = base_vocab; L.fim_suffix = base_vocab + 1; L.fim_middle = base_vocab + 2; L.fim_pad = base_vocab + 3;
  L.fim_rate = rate;
  L.spm_rate = spm_rate;
  return 0;
}

int eisen_loader_seed(void* h, unsigned long long seed) {
  if (!h) { set_error("loader_seed: null handle"); return EISEN_ERR_INVALID; }
  H(h)->rng.s = seed;
  return 0;
}

int eisen_loader_reset(void* h) {  // dataloader.rs:196-199 (the generator keeps its state)
  if (!h) { set_error("loader_reset: null handle"); return EISEN_ERR_INVALID; }
  Loader& L = *H(h);
  fseek(L.f, 0, SEEK_SET);
  L.buffer.clear();
  L.head = 0;
  return 0;
}

// Fills x[batch * seq_len] and targets[batch * seq_len]; *has_masked (may be null) is set when a
// target is the ignore index.  Returns 0, or 1 when the file has no complete batch left.
int eisen_loader_next(void* h, int* x, int* targets, int* has_masked) {
  if (!h || !x || !targets) { set_error("loader_next: null argument"); return EISEN_ERR_INVALID; }
  Loader& L = *H(h);
  const size_t need = (size_t)(L.batch * (L.seq_len + 1));
  if (L.buffer.size() - L.head < need) {  // refill: 100 batches' worth per read (dataloader.rs:137-150)
    L.buffer.erase(L.buffer.begin(), L.buffer.begin() + (long long)L.head);
    L.head = 0;
    std::vector<uint8_t> bytes(need * 100 * 2);
    const size_t got = fread(bytes.data(), 1, bytes.size(), L.f);
    const size_t ntok = got / 2;
    const size_t old = L.buffer.size();
    L.buffer.resize(old + ntok);
    for (size_t i = 0; i < ntok; ++i) L.buffer[old + i] = (int32_t)((uint32_t)bytes[2 * i] | ((uint32_t)bytes[2 * i + 1] << 8));
    if (L.buffer.size() < need) return 1;
  }
  bool masked = false;
  std::vector<uint8_t> mask((size_t)L.seq_len);
  std::vector<int32_t> fx((size_t)L.seq_len);
  for (long long b = 0; b < L.batch; ++b) {
    const int32_t* raw = L.buffer.data() + L.head + (size_t)(b * (L.seq_len + 1));
    int32_t* xo = x + b * L.seq_len;
    int32_t* yo = targets + b * L.seq_len;
    const float draw = L.rng.unit_f32();  // drawn for every sequence, FIM or not
    if (L.fim && draw < L.fim_rate) {
      apply_fim(raw, L.seq_len, L, L.rng, fx.data(), mask.data());
      // y[i] = x'[i + 1], the last position has no successor; positions whose mask is off are
      // ignored (dataloader.rs:170-181, fim.rs:174-179: the mask of position i itself is used)
      for (long long i = 0; i < L.seq_len; ++i) {
        xo[i] = fx[(size_t)i];
        const int32_t y = i + 1 < L.seq_len ? fx[(size_t)i + 1] : IGNORE;
        yo[i] = mask[(size_t)i] ? y : IGNORE;
      }
      masked = true;  // dataloader.rs:183: set for every transformed sequence
    } else {
      for (long long i = 0; i < L.seq_len; ++i) { xo[i] = raw[i]; yo[i] = raw[i + 1]; }
    }
  }
  L.head += need;
  if (has_masked) *has_masked = masked ? 1 : 0;
  return 0;
}

}  // extern "C"
