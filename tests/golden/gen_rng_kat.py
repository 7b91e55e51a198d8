"""Generates tests/golden/rng_kat.json.

An independent restatement of the reference's RNG contract with Python
integers only (no shared code with the C oracle or the CUDA library):
  noise_seed            hyperscalees-noiser/src/noiser.rs:495-506
  xorshift64 / unit     noiser.rs:444-460
  standard_normal       noiser.rs:470-477 (libm logf/cosf/sqrtf through ctypes)
  epoch_thread_sign     hyperscalees-noiser/src/eggroll.rs:60-65
  xorshift32 Poisson    hyperscalees-kernels/src/poisson_encode_fused_oxide.rs:36-52,84-105
  taus88+LCG stream     hyperscalees-kernels/src/lib.rs:26-101
The float values depend on the host libm (glibc x86-64 here); the integer
streams do not.  Run: python tests/golden/gen_rng_kat.py
"""
import ctypes
import json
import os
import struct

libm = ctypes.CDLL("libm.so.6")
for f in ("logf", "cosf", "sinf", "sqrtf"):
    getattr(libm, f).restype = ctypes.c_float
    getattr(libm, f).argtypes = [ctypes.c_float]
M64 = (1 << 64) - 1
M32 = (1 << 32) - 1


def f32(x):
    return struct.unpack("f", struct.pack("f", x))[0]


def bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def sext(v):
    return v & M64


def noise_seed(key, te, tt):
    h = key ^ 0x9E3779B97F4A7C15
    h = (h * 0xBF58476D1CE4E5B9) & M64
    h ^= (sext(te) * 0x94D049BB133111EB) & M64
    h = (((h << 17) | (h >> 47)) & M64) ^ sext(tt)
    h ^= h >> 33
    h = (h * 0xBF58476D1CE4E5B9) & M64
    h ^= h >> 29
    h = (h * 0x94D049BB133111EB) & M64
    h ^= h >> 32
    return h


class Stream:
    def __init__(self, seed):
        self.s = seed | 1

    def u64(self):
        x = self.s
        x ^= (x << 13) & M64
        x ^= x >> 7
        x ^= (x << 17) & M64
        self.s = x
        return x

    def unit(self):
        return f32((self.u64() >> 40) / float(1 << 24))

    def normal(self):
        u1 = max(self.unit(), f32(1e-9))
        u2 = self.unit()
        rad = libm.sqrtf(f32(-2.0 * libm.logf(u1)))
        th = f32(f32(6.283185307179586) * u2)
        return f32(rad * libm.cosf(th))


def xs32(x):
    x ^= (x << 13) & M32
    x ^= x >> 17
    x ^= (x << 5) & M32
    return x


def taus(z, s1, s2, s3, m):
    b = ((((z << s1) & M32) ^ z) >> s2)
    return (((z & m) << s3) & M32) ^ b


def main():
    out = {"noise_seed": [], "streams": [], "poisson": [], "taus": []}
    key_mul = 0x9E3779B97F4A7C15
    keys = [((i + 1) * key_mul) & M64 for i in range(4)] + [7, 5, 99, 0, M64]
    for key in keys:
        for te, tt in [(0, 0), (0, 1), (3, 5), (-1, 2), (7, -3), (0, 32767)]:
            out["noise_seed"].append({"key": str(key), "te": te, "tt": tt, "seed": str(noise_seed(key, te, tt))})
    for key, te, tt in [(keys[0], 0, 0), (keys[0], 0, 1), (keys[0], 3, 5), (keys[1], 0, 0), (keys[1], 0, 1),
                        (keys[1], 3, 5), (7, 0, 0), (99, 0, 0)]:
        seed = noise_seed(key, te, tt)
        s = Stream(seed)
        u = [str(s.u64()) for _ in range(8)]
        s = Stream(seed)
        n = [bits(s.normal()) for _ in range(64)]
        out["streams"].append({"key": str(key), "te": te, "tt": tt, "seed": str(seed), "u64": u, "normal_bits": n})
    for idx, mix in [(0, 0), (1, 0), (12345, 0xDEADBEEF), (783, 1), (2 ** 31 + 5, 42)]:
        x = (1000000007 * idx + mix + 0x9E3779B9) & M32
        ks = []
        for _ in range(8):
            x = xs32(x)
            ks.append((x >> 9) + 1)
        out["poisson"].append({"idx": idx, "mix": mix, "n": ks,
                               "u_bits": [bits(f32(f32(float(k)) / f32(8388609.0))) for k in ks]})
    for t, seeds in [(0, (1, 2, 3, 4)), (5, (11, 22, 33, 44)), (1000, (0xFFFFFFFF, 7, 0, 9))]:
        s = (1000000007 * t) & M32
        st = [(s + sd) & M32 for sd in seeds]
        ints = []
        for _ in range(8):
            st[0] = taus(st[0], 13, 19, 12, 4294967294)
            st[1] = taus(st[1], 2, 25, 4, 4294967288)
            st[2] = taus(st[2], 3, 11, 17, 4294967280)
            st[3] = (st[3] * 1664525 + 1013904223) & M32
            ints.append(st[0] ^ st[1] ^ st[2] ^ st[3])
        out["taus"].append({"thread": t, "seeds": list(seeds), "ints": ints})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rng_kat.json")
    with open(path, "w") as fh:
        json.dump(out, fh, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
