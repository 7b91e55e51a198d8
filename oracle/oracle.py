"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only the test suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the shipped package never does.  `build()` compiles
`hses_oracle.c` next to this file with the Makefile beside it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libhses_oracle.so")
_lib = None

RESET_HARD, RESET_SUBTRACT = 0, 1
REWARD_LOGLIK, REWARD_BINARY = 0, 1
SGD, ADAM, ADAMW = 0, 1, 2

_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_u64p = C.POINTER(C.c_uint64)
_u32p = C.POINTER(C.c_uint32)
_u8p = C.POINTER(C.c_uint8)


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "hses_oracle.c")
    hdr = os.path.join(_HERE, "hses_oracle.h")
    stale = (not os.path.exists(_SO)) or any(
        os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(_SO) for p in (src, hdr)
    )
    if force or stale:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return _SO


class _Snn(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int),
        ("dims", C.POINTER(C.c_int)),
        ("w", C.POINTER(_f32p)),
        ("keys", _u64p),
        ("out_gain", C.c_float),
        ("tau_m", C.c_float),
        ("v_th", C.c_float),
        ("v_th_layer", _f32p),
        ("reset_mode", C.c_int),
        ("sigma", C.c_float),
        ("rank", C.c_int),
        ("noise_reuse", C.c_int32),
    ]


class _Solver(C.Structure):
    _fields_ = [("kind", C.c_int), ("lr", C.c_float), ("beta1", C.c_float),
                ("beta2", C.c_float), ("eps", C.c_float), ("weight_decay", C.c_float)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.hso_noise_seed.restype = C.c_uint64
        L.hso_noise_seed.argtypes = [C.c_uint64, C.c_int32, C.c_int32]
        L.hso_clip_scale.restype = C.c_float
        L.hso_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_i32p)


def num_threads() -> int:
    return int(lib().hso_num_threads())


def set_num_threads(n: int) -> None:
    lib().hso_set_num_threads(int(n))


def noise_seed(key: int, true_epoch: int, true_thread: int) -> int:
    return int(lib().hso_noise_seed(C.c_uint64(key & (2**64 - 1)), true_epoch, true_thread))


def xorshift64_stream(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint64)
    lib().hso_xorshift64_stream(C.c_uint64(seed), out.ctypes.data_as(_u64p), C.c_size_t(n))
    return out


def units(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().hso_units(C.c_uint64(seed), out.ctypes.data_as(_f32p), C.c_size_t(n))
    return out


def normals(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().hso_normals(C.c_uint64(seed), out.ctypes.data_as(_f32p), C.c_size_t(n))
    return out


def epoch_thread_sign(epoch: int, thread_id: int, noise_reuse: int):
    te, tt, sg = C.c_int32(), C.c_int32(), C.c_float()
    lib().hso_epoch_thread_sign(epoch, thread_id, noise_reuse, C.byref(te), C.byref(tt), C.byref(sg))
    return te.value, tt.value, sg.value


def lora_params(base_sigma: float, key: int, rank: int, epoch: int, thread_id: int,
                a: int, b: int, noise_reuse: int):
    A = np.empty((a, rank), dtype=np.float32)
    B = np.empty((b, rank), dtype=np.float32)
    lib().hso_lora_params(C.c_float(base_sigma), C.c_uint64(key), rank, epoch, thread_id, a, b,
                          noise_reuse, A.ctypes.data_as(_f32p), B.ctypes.data_as(_f32p))
    return A, B


def nonlora_params(base_sigma: float, key: int, epoch: int, thread_id: int, rows: int,
                   cols: int, noise_reuse: int) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float32)
    lib().hso_nonlora_params(C.c_float(base_sigma), C.c_uint64(key), epoch, thread_id, rows, cols,
                             noise_reuse, out.ctypes.data_as(_f32p))
    return out


def do_mm(x, param, sigma: float, rank: int, key: int, iterinfo=None, noise_reuse: int = 0,
          acc64: bool = False) -> np.ndarray:
    x, xp = _f(x)
    param, pp = _f(param)
    bm, b = x.shape
    a = param.shape[0]
    assert param.shape[1] == b
    y = np.empty((bm, a), dtype=np.float32)
    ep, tid = iterinfo if iterinfo is not None else (0, 0)
    lib().hso_do_mm(xp, bm, pp, a, b, C.c_float(sigma), rank, C.c_uint64(key),
                    int(iterinfo is not None), ep, tid, noise_reuse, int(acc64),
                    y.ctypes.data_as(_f32p))
    return y


def run_lif(cur, v0, tau_m: float, v_th: float, reset_mode: int = RESET_HARD):
    cur, cp = _f(cur)
    T = cur.shape[0]
    nh = int(np.prod(cur.shape[1:]))
    v = np.array(v0, dtype=np.float32, copy=True).reshape(-1)
    assert v.size == nh
    sp = np.empty_like(cur)
    lib().hso_run_lif(cp, T, C.c_size_t(nh), C.c_float(tau_m), C.c_float(v_th), reset_mode,
                      v.ctypes.data_as(_f32p), sp.ctypes.data_as(_f32p))
    return sp, v.reshape(cur.shape[1:])


def poisson_encode(probs, T: int, seeds: Sequence[int]):
    """probs is a dense (batch, in_dim) matrix; returns (T, batch, in_dim)."""
    return poisson_encode_pitched(probs, np.asarray(probs).shape[1], T, seeds)


def poisson_encode_pitched(probs_pitched, in_dim: int, T: int, seeds: Sequence[int]):
    """probs_pitched is (batch, row_stride) with only the first in_dim columns used."""
    probs, pp = _f(probs_pitched)
    batch, stride = probs.shape
    out = np.zeros((T, batch, stride), dtype=np.float32)
    sd = (C.c_uint32 * 4)(*[int(s) & 0xFFFFFFFF for s in seeds])
    lib().hso_poisson_encode(pp, C.c_size_t(batch), C.c_size_t(in_dim), C.c_size_t(stride), T,
                             sd, out.ctypes.data_as(_f32p))
    return out


def fitness(logits, labels, reward: int = REWARD_LOGLIK) -> np.ndarray:
    logits, lp = _f(logits)
    labels, bp = _i(labels)
    n, c = logits.shape
    out = np.empty(n, dtype=np.float32)
    lib().hso_fitness(lp, C.c_size_t(n), c, bp, reward, out.ctypes.data_as(_f32p))
    return out


def convert_fitnesses_bs(raw, group_size: int) -> np.ndarray:
    raw, rp = _f(raw)
    out = np.empty(group_size, dtype=np.float32)
    lib().hso_convert_fitnesses_bs(rp, C.c_size_t(raw.size), group_size, out.ctypes.data_as(_f32p))
    return out


def convert_fitnesses(raw, group_size: int = 0) -> np.ndarray:
    raw, rp = _f(raw)
    out = np.empty_like(raw)
    lib().hso_convert_fitnesses(rp, C.c_size_t(raw.size), group_size, out.ctypes.data_as(_f32p))
    return out


@dataclass
class Snn:
    """Host description of an SNN MLP: weights are (out, in) row-major."""
    weights: Sequence[np.ndarray]
    keys: Sequence[int]
    out_gain: float = 1.0
    tau_m: float = 20.0
    v_th: float = 0.3
    v_th_layer: Optional[Sequence[float]] = None
    reset_mode: int = RESET_HARD
    sigma: float = 0.02
    rank: int = 4
    noise_reuse: int = 0
    _keep: list = field(default_factory=list, repr=False)

    def _struct(self):
        ws = [np.ascontiguousarray(w, dtype=np.float32) for w in self.weights]
        dims = [ws[0].shape[1]] + [w.shape[0] for w in ws]
        dims_c = (C.c_int * len(dims))(*dims)
        wp = (_f32p * len(ws))(*[w.ctypes.data_as(_f32p) for w in ws])
        keys = (C.c_uint64 * len(ws))(*[int(k) & (2**64 - 1) for k in list(self.keys)[:len(ws)]])
        vl = None
        if self.v_th_layer is not None:
            vl = (C.c_float * len(self.v_th_layer))(*self.v_th_layer)
        s = _Snn(len(ws), dims_c, wp, keys, self.out_gain, self.tau_m, self.v_th,
                 C.cast(vl, _f32p) if vl is not None else None, self.reset_mode, self.sigma,
                 self.rank, self.noise_reuse)
        self._keep = [ws, dims_c, wp, keys, vl]
        return s, dims

    def forward(self, spikes_in, iterinfo=None, acc64: bool = False, want_hidden: bool = False):
        s, dims = self._struct()
        x, xp = _f(spikes_in)
        T, bm, _ = x.shape
        logits = np.empty((bm, dims[-1]), dtype=np.float32)
        hid = np.empty((T, bm, dims[-2]), dtype=np.float32) if want_hidden else None
        ep, tid = iterinfo if iterinfo is not None else (0, 0)
        lib().hso_snn_forward(C.byref(s), xp, T, bm, int(iterinfo is not None), ep, tid,
                              int(acc64), logits.ctypes.data_as(_f32p),
                              hid.ctypes.data_as(_f32p) if want_hidden else None)
        return (logits, hid) if want_hidden else logits


def lora_grad(sigma, key, a, b, rank, scores, epochs, thread_ids, noise_reuse=0):
    scores, sp = _f(scores)
    epochs, ep = _i(epochs)
    tids, tp = _i(thread_ids)
    out = np.empty((a, b), dtype=np.float32)
    lib().hso_lora_grad(C.c_float(sigma), C.c_uint64(key), a, b, rank, sp, ep, tp,
                        C.c_size_t(scores.size), noise_reuse, out.ctypes.data_as(_f32p))
    return out



def lora_grad_block(sigma, key, a, b, rank, scores, epochs, thread_ids, rows, cols, noise_reuse=0):
    """Rows [rows[0], rows[1]) x columns [cols[0], cols[1]) of lora_grad, member sum in fp64."""
    scores, sp = _f(scores)
    epochs, ep = _i(epochs)
    tids, tp = _i(thread_ids)
    out = np.empty((rows[1] - rows[0], cols[1] - cols[0]), dtype=np.float32)
    lib().hso_lora_grad_block(C.c_float(sigma), C.c_uint64(key), a, b, rank, sp, ep, tp,
                              C.c_size_t(scores.size), noise_reuse, rows[0], rows[1], cols[0], cols[1],
                              out.ctypes.data_as(_f32p))
    return out


def alt_lora_grad(sigma, key, a, b, rank, scores, epochs, thread_ids, noise_reuse=0):
    scores, sp = _f(scores)
    epochs, ep = _i(epochs)
    tids, tp = _i(thread_ids)
    out = np.empty((a, b), dtype=np.float32)
    lib().hso_alt_lora_grad(C.c_float(sigma), C.c_uint64(key), a, b, rank, sp, ep, tp,
                        C.c_size_t(scores.size), noise_reuse, out.ctypes.data_as(_f32p))
    return out

def full_grad(sigma, key, rows, cols, scores, epochs, thread_ids, noise_reuse=0,
              freeze_nonlora=False):
    scores, sp = _f(scores)
    epochs, ep = _i(epochs)
    tids, tp = _i(thread_ids)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().hso_full_grad(C.c_float(sigma), C.c_uint64(key), rows, cols, sp, ep, tp,
                        C.c_size_t(scores.size), noise_reuse, int(freeze_nonlora),
                        out.ctypes.data_as(_f32p))
    return out


def lora_einsum_raw(a_t, b_t, scores):
    a_t, ap = _f(a_t)
    b_t, bp = _f(b_t)
    scores, sp = _f(scores)
    n, r, a = a_t.shape
    b = b_t.shape[2]
    out = np.empty((a, b), dtype=np.float32)
    lib().hso_lora_einsum_raw(ap, bp, sp, C.c_size_t(n), r, a, b, out.ctypes.data_as(_f32p))
    return out


def lora_einsum_ones(a_t, b_t):
    a_t, ap = _f(a_t)
    b_t, bp = _f(b_t)
    n, r, a = a_t.shape
    b = b_t.shape[2]
    out = np.empty((a, b), dtype=np.float32)
    lib().hso_lora_einsum_ones(ap, bp, C.c_size_t(n), r, a, b, out.ctypes.data_as(_f32p))
    return out


def lora_einsum_pair_half(a_half, b_half, scores):
    a_half, ap = _f(a_half)
    b_half, bp = _f(b_half)
    scores, sp = _f(scores)
    half, r, a = a_half.shape
    b = b_half.shape[2]
    g_raw = np.empty((a, b), dtype=np.float32)
    g_ones = np.empty((a, b), dtype=np.float32)
    lib().hso_lora_einsum_pair_half(ap, bp, sp, C.c_size_t(half), r, a, b,
                                    g_raw.ctypes.data_as(_f32p), g_ones.ctypes.data_as(_f32p))
    return g_raw, g_ones


def combine_affine(grad_acc, ones_acc, mean, std, batch):
    g, gp = _f(grad_acc)
    o, op = _f(ones_acc)
    out = np.empty_like(g)
    lib().hso_combine_affine(gp, op, C.c_size_t(g.size), C.c_float(mean), C.c_float(std),
                             C.c_size_t(batch), out.ctypes.data_as(_f32p))
    return out


def solver_update(kind, step, param, grad, m=None, v=None, lr=0.01, beta1=0.9, beta2=0.999,
                  eps=1e-8, weight_decay=0.0):
    s = _Solver(kind, lr, beta1, beta2, eps, weight_decay)
    p = np.array(param, dtype=np.float32, copy=True)
    g, gp = _f(grad)
    m = np.zeros_like(p) if m is None else np.array(m, dtype=np.float32, copy=True)
    v = np.zeros_like(p) if v is None else np.array(v, dtype=np.float32, copy=True)
    lib().hso_solver_update(C.byref(s), step, p.ctypes.data_as(_f32p), gp,
                            m.ctypes.data_as(_f32p), v.ctypes.data_as(_f32p), C.c_size_t(p.size))
    return p, m, v


def clip_scale(grads, max_norm: float) -> float:
    arrs = [np.ascontiguousarray(g, dtype=np.float32) for g in grads]
    ptrs = (_f32p * len(arrs))(*[a.ctypes.data_as(_f32p) for a in arrs])
    lens = (C.c_size_t * len(arrs))(*[a.size for a in arrs])
    return float(lib().hso_clip_scale(ptrs, lens, len(arrs), C.c_float(max_norm)))


def perturbed_linear_lif(x, param, sigma, rank, key, epoch=0, first_thread=0, noise_reuse=0,
                         tau_m=20.0, v_th=0.3, reset_mode=RESET_HARD, acc64=False,
                         want_potentials=False):
    x, xp = _f(x)
    param, pp = _f(param)
    n_pop, bm, k = x.shape
    a = param.shape[0]
    sp = np.empty((n_pop, bm, a), dtype=np.float32)
    pot = np.empty((n_pop, bm, a), dtype=np.float32) if want_potentials else None
    lib().hso_perturbed_linear_lif(xp, C.c_size_t(n_pop), bm, k, pp, a, C.c_float(sigma), rank,
                                   C.c_uint64(key), epoch, first_thread, noise_reuse,
                                   C.c_float(tau_m), C.c_float(v_th), reset_mode, int(acc64),
                                   sp.ctypes.data_as(_f32p),
                                   pot.ctypes.data_as(_f32p) if want_potentials else None)
    return (sp, pot) if want_potentials else sp


def prng_normal_half(total_threads: int, mean: float, std: float, seeds: Sequence[int]):
    out = np.empty(total_threads * 128, dtype=np.float32)
    sd = (C.c_uint32 * 4)(*[int(s) & 0xFFFFFFFF for s in seeds])
    lib().hso_prng_normal_half(out.ctypes.data_as(_f32p), C.c_size_t(total_threads),
                               C.c_float(mean), C.c_float(std), sd)
    return out


def wkv7(r, w, k, v, a, b, state, new_starts=None):
    r, rp = _f(r); w, wp = _f(w); k, kp = _f(k); v, vp = _f(v); a, ap = _f(a); b, bp = _f(b)
    T, H, S = r.shape
    st = np.array(state, dtype=np.float32, copy=True)
    out = np.empty((T, H, S), dtype=np.float32)
    ns = None
    if new_starts is not None:
        ns = np.ascontiguousarray(new_starts, dtype=np.uint8)
    lib().hso_wkv7(rp, wp, kp, vp, ap, bp, ns.ctypes.data_as(_u8p) if ns is not None else None,
                   T, H, S, st.ctypes.data_as(_f32p), out.ctypes.data_as(_f32p))
    return st, out


def spiking_attention(Q, K, V, mode=0, beta=1.0, tau_m=2.0, v_th=0.3, g_inh=0.5, n_iter=8):
    """One head: Q, K, V (tokens, d) -> (O (tokens, d), A (tokens, tokens))."""
    Q, qp = _f(Q); K, kp = _f(K); V, vp = _f(V)
    tokens, d = Q.shape
    O = np.empty((tokens, d), dtype=np.float32)
    A = np.empty((tokens, tokens), dtype=np.float32)
    lib().hso_spiking_attention(qp, kp, vp, tokens, d, mode, C.c_float(beta), C.c_float(tau_m), C.c_float(v_th),
                                C.c_float(g_inh), n_iter, O.ctypes.data_as(_f32p), A.ctypes.data_as(_f32p))
    return O, A


def layer_norm(x, weight, bias, eps=1e-5):
    x, xp = _f(x); w, wp = _f(weight); b, bp = _f(bias)
    c = x.shape[-1]
    out = np.empty_like(x)
    lib().hso_layer_norm(xp, C.c_size_t(x.size // c), c, wp, bp, C.c_float(eps), out.ctypes.data_as(_f32p))
    return out


def group_norm(x, groups, weight, bias, eps=1e-5):
    """x (n, c) or (n, c, l)."""
    x, xp = _f(x); w, wp = _f(weight); b, bp = _f(bias)
    n, c = x.shape[0], x.shape[1]
    l = x.shape[2] if x.ndim == 3 else 1
    out = np.empty_like(x)
    lib().hso_group_norm(xp, C.c_size_t(n), c, l, groups, wp, bp, C.c_float(eps), out.ctypes.data_as(_f32p))
    return out


def token_shift_mix(x, state, coef, new_starts=None):
    x, xp = _f(x); st, sp = _f(state); cf, cp = _f(coef)
    T, c = x.shape
    ns = np.ascontiguousarray(new_starts, dtype=np.uint8) if new_starts is not None else None
    out = np.empty_like(x)
    lib().hso_token_shift_mix(xp, T, c, sp, ns.ctypes.data_as(_u8p) if ns is not None else None, cp,
                              out.ctypes.data_as(_f32p))
    return out


def channel_mix(x, state, x_k, wk, wv, length, new_starts=None):
    """ChannelMixing.forward: returns (out (T, c), state_out (c,))."""
    x, xp = _f(x); st, sp = _f(state); xk, xkp = _f(x_k); wk, wkp = _f(wk); wv, wvp = _f(wv)
    T, c = x.shape
    f = wk.shape[0]
    ns = np.ascontiguousarray(new_starts, dtype=np.uint8) if new_starts is not None else None
    out = np.empty_like(x)
    so = np.empty(c, dtype=np.float32)
    lib().hso_channel_mix(xp, T, c, f, sp, ns.ctypes.data_as(_u8p) if ns is not None else None, xkp, wkp, wvp,
                          length, out.ctypes.data_as(_f32p), so.ctypes.data_as(_f32p))
    return out, so


def rate_encode(p, gain):
    p, pp = _f(p)
    out = np.empty_like(p)
    lib().hso_rate_encode(pp, C.c_size_t(p.size), C.c_float(gain), out.ctypes.data_as(_f32p))
    return out
