"""CPU restatement of the reference's BinaryDataLoader and FIM transform (test infrastructure only).

Follows src/data/dataloader.rs:96-207 and src/data/fim.rs:96-180 statement by statement with Python
integers (u64 arithmetic masked by hand).  The integer-range and f32 sampling rules are those of the
`rand` crate the reference pins (rand 0.8.5, Cargo.lock): UniformInt::sample_single (widening
multiply with rejection zone) and Standard for f32 (top 24 bits of a u32).  The reference has no test
for this path, so parity with it is pinned by restatement only.

Only tests may import this file; the product reads files through libeisen_b200.so (eisen_loader_*).
"""
import numpy as np

M64 = (1 << 64) - 1
IGNORE_INDEX = -1  # the reference uses usize::MAX; the device path takes -1


class XorShift64:
    """dataloader.rs:201-207 (xorshift_f32) and 214-221 (the RngCore adapter)."""

    def __init__(self, seed):
        self.s = seed & M64

    def next_u64(self):
        s = self.s
        s ^= (s << 13) & M64
        s ^= s >> 7
        s ^= (s << 17) & M64
        self.s = s
        return s

    def unit_f32(self):
        # (state >> 11) as f32 / (1u64 << 53) as f32
        return np.float32(np.float32(self.next_u64() >> 11) / np.float32(1 << 53))

    def gen_f32(self):
        # rand 0.8.5 Standard<f32>: value: u32 = next_u32(); (value >> 8) as f32 * 2^-24
        v = self.next_u64() & 0xFFFFFFFF
        return np.float32(np.float32(v >> 8) * np.float32(1.0 / (1 << 24)))

    def gen_range(self, low, high):
        # rand 0.8.5 UniformInt<usize>::sample_single(low, high): range = high - low;
        # zone = (range << range.leading_zeros()) - 1; accept when the low word <= zone
        rng = high - low
        assert rng > 0
        lz = 64 - rng.bit_length()
        zone = ((rng << lz) & M64) - 1
        while True:
            m = self.next_u64() * rng
            hi, lo = m >> 64, m & M64
            if lo <= zone:
                return low + hi


def apply_fim(tokens, prefix_id, suffix_id, middle_id, pad_id, spm_rate, rng, seq_len):
    """fim.rs:96-168 -> (tokens', mask)."""
    n = len(tokens)
    if n < 4:
        out = list(tokens) + [pad_id] * (seq_len - n)
        return out[:seq_len], [True] * seq_len
    lo = rng.gen_range(1, n - 2)
    hi = rng.gen_range(lo + 1, n - 1)
    prefix, middle, suffix = tokens[:lo], tokens[lo:hi], tokens[hi:]
    use_spm = rng.gen_f32() < np.float32(spm_rate)
    res, mask = [], []
    if use_spm:
        parts = [([suffix_id], False), (suffix, False), ([prefix_id], False), (prefix, False)]
    else:
        parts = [([prefix_id], False), (prefix, False), ([suffix_id], False), (suffix, False)]
    parts += [([middle_id], False), (middle, True)]
    for seg, m in parts:
        res.extend(seg)
        mask.extend([m] * len(seg))
    res, mask = res[:seq_len], mask[:seq_len]
    while len(res) < seq_len:
        res.append(pad_id)
        mask.append(False)
    return res, mask


class BinaryDataLoaderOracle:
    """dataloader.rs:96-199.  next_batch() -> (x[int32], targets[int32], has_masked) or None."""

    def __init__(self, path, seq_len, batch, fim=None, seed=1337):
        self.tokens = np.fromfile(path, dtype="<u2").astype(np.int64)
        self.seq_len, self.batch = seq_len, batch
        self.fim = fim  # None or (base_vocab, rate, spm_rate)
        self.rng = XorShift64(seed)
        self.pos = 0
        self.total_batches = len(self.tokens) // (batch * (seq_len + 1))

    def reset(self):
        self.pos = 0

    def next_batch(self):
        need = self.batch * (self.seq_len + 1)
        if len(self.tokens) - self.pos < need:
            return None
        buf = self.tokens[self.pos:self.pos + need]
        xs, ys, has_masked = [], [], False
        for b in range(self.batch):
            start = b * (self.seq_len + 1)
            raw_x = [int(t) for t in buf[start:start + self.seq_len]]
            raw_y = [int(t) for t in buf[start + 1:start + self.seq_len + 1]]
            draw = self.rng.unit_f32()
            if self.fim is not None and draw < np.float32(self.fim[1]):
                base, _, spm = self.fim
                fx, mask = apply_fim(raw_x, base, base + 1, base + 2, base + 3, spm, self.rng, self.seq_len)
                fy = fx[1:] + [IGNORE_INDEX]
                fy = [t if m else IGNORE_INDEX for t, m in zip(fy, mask)]
                has_masked = True
                xs.extend(fx)
                ys.extend(fy)
            else:
                xs.extend(raw_x)
                ys.extend(raw_y)
        self.pos += need
        return np.asarray(xs, dtype=np.int32), np.asarray(ys, dtype=np.int32), has_masked
