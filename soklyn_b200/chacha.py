"""ChaCha8 random generator as the reference's weight initialisers use it
(src/util/function.rs:219-248: `rand_chacha::ChaCha8Rng::seed_from_u64(seed)`, then `next_u32`).

rand_chacha 0.9.0 and rand_core 0.9 are dependencies the reference pins in Cargo.lock; their sources
are not part of the reference tree, so this restates the published algorithms:

* the ChaCha block function with 8 rounds (Bernstein's ChaCha; constants "expand 32-byte k", eight
  key words, a 64-bit block counter in words 12-13 and a 64-bit stream id, zero, in words 14-15);
  the generator's output is the keystream read as little-endian 32-bit words, block after block
  from counter 0;
* `SeedableRng::seed_from_u64`: the 32-byte key is eight outputs of a PCG32 generator (multiplier
  6364136223846793005, increment 11634580027462260723, state advanced before each output,
  XSH-RR output function) started from the given 64-bit value.

The block function is pinned by the 8-round known-answer vector for the all-zero key and nonce
(tests/test_host_cpu.py). The seed expansion and the pairing of draws have no vector to be checked
against here.
"""
from __future__ import annotations

import numpy as np

_CONSTANTS = np.array([0x61707865, 0x3320646E, 0x79622D32, 0x6B206574], dtype=np.uint32)
_MASK64 = (1 << 64) - 1


def _rotl(x: np.ndarray, n: int) -> np.ndarray:
    return (x << np.uint32(n)) | (x >> np.uint32(32 - n))


def _quarter(s, a, b, c, d):
    s[a] += s[b]; s[d] = _rotl(s[d] ^ s[a], 16)
    s[c] += s[d]; s[b] = _rotl(s[b] ^ s[c], 12)
    s[a] += s[b]; s[d] = _rotl(s[d] ^ s[a], 8)
    s[c] += s[d]; s[b] = _rotl(s[b] ^ s[c], 7)


def chacha_blocks(key_words: np.ndarray, first_block: int, count: int, rounds: int = 8) -> np.ndarray:
    """Keystream words of blocks [first_block, first_block + count): uint32 array [count, 16]."""
    counters = np.arange(first_block, first_block + count, dtype=np.uint64)
    init = [np.full(count, _CONSTANTS[i], dtype=np.uint32) for i in range(4)]
    init += [np.full(count, np.uint32(key_words[i]), dtype=np.uint32) for i in range(8)]
    init += [(counters & np.uint64(0xFFFFFFFF)).astype(np.uint32), (counters >> np.uint64(32)).astype(np.uint32),
             np.zeros(count, np.uint32), np.zeros(count, np.uint32)]
    s = [w.copy() for w in init]
    with np.errstate(over="ignore"):
        for _ in range(rounds // 2):
            _quarter(s, 0, 4, 8, 12); _quarter(s, 1, 5, 9, 13); _quarter(s, 2, 6, 10, 14); _quarter(s, 3, 7, 11, 15)
            _quarter(s, 0, 5, 10, 15); _quarter(s, 1, 6, 11, 12); _quarter(s, 2, 7, 8, 13); _quarter(s, 3, 4, 9, 14)
        out = np.stack([a + b for a, b in zip(s, init)], axis=1)
    return out


def seed_words_from_u64(seed: int) -> np.ndarray:
    """rand_core's seed_from_u64: eight PCG32 (XSH-RR) outputs."""
    state, words = seed & _MASK64, []
    for _ in range(8):
        state = (state * 6364136223846793005 + 11634580027462260723) & _MASK64
        xorshifted = (((state >> 18) ^ state) >> 27) & 0xFFFFFFFF
        rot = state >> 59
        words.append(((xorshifted >> rot) | (xorshifted << ((32 - rot) & 31))) & 0xFFFFFFFF)
    return np.array(words, dtype=np.uint32)


class ChaCha8Rng:
    """Sequential 32-bit draws from the ChaCha8 keystream of a key."""

    def __init__(self, key_words):
        self.key = np.asarray(key_words, dtype=np.uint32)
        self.pos = 0   # index of the next 32-bit word in the stream

    @staticmethod
    def seed_from_u64(seed: int) -> "ChaCha8Rng":
        return ChaCha8Rng(seed_words_from_u64(seed))

    def next_u32s(self, n: int) -> np.ndarray:
        """The next n draws of next_u32, as a uint32 array."""
        first, last = self.pos // 16, (self.pos + n + 15) // 16
        out = np.empty(n, dtype=np.uint32)
        done, chunk = 0, 1 << 18    # blocks per batch: bounded temporaries
        for b0 in range(first, last, chunk):
            words = chacha_blocks(self.key, b0, min(chunk, last - b0)).reshape(-1)
            lo = self.pos - b0 * 16 if b0 == first else 0
            take = min(n - done, words.size - lo)
            out[done:done + take] = words[lo:lo + take]
            done += take
        self.pos += n
        return out

    def next_u32(self) -> int:
        return int(self.next_u32s(1)[0])
