"""Generates tests/golden/wkv7_golden.json: a WKV-7 recurrence case with non-zero k, v, a and b.

The recurrence is restated here in plain numpy from its published form, following the order of
operations of the reference's loop (src/hyperscalees/models/llm/rwkv7.py:200-220, `inner_loop`;
the Rust port hyperscalees-models/src/llm.rs:235-296 is the same algebra): per step and head

    w   = exp(-exp(w_in))
    sa  = S @ a                      (S is (S, S), a a column)
    S   = S * w[None, :] + v[:, None] @ k[None, :] + sa[:, None] @ b[None, :]
    out = S @ r

with a state reset where new_starts is set, all in float64 (the fixture is the mathematical value;
the fp32 implementations are held to 1e-5 of it).  Inputs are drawn from a seeded generator and
written out with the results, so the test needs neither this script nor numpy's generator.

    python tests/golden/gen_wkv7_golden.py
"""
import json
import os

import numpy as np


def wkv7(r, w, k, v, a, b, s0, new_starts):
    T, H, S = r.shape
    s = s0.astype(np.float64).copy()
    out = np.zeros((T, H, S), np.float64)
    wd = np.exp(-np.exp(w.astype(np.float64)))
    for t in range(T):
        if new_starts[t]:
            s[:] = 0.0
        for h in range(H):
            sa = s[h] @ a[t, h].astype(np.float64)
            s[h] = s[h] * wd[t, h][None, :] + np.outer(v[t, h], k[t, h]) + np.outer(sa, b[t, h])
            out[t, h] = s[h] @ r[t, h].astype(np.float64)
    return s, out


def main():
    g = np.random.Generator(np.random.PCG64(77))
    T, H, S = 6, 2, 4
    mk = lambda sc: (g.standard_normal((T, H, S)) * sc).astype(np.float32)
    r, k, v, a, b = mk(1.0), mk(0.5), mk(1.0), mk(0.3), mk(0.3)
    w = (g.standard_normal((T, H, S)) * 0.5 - 1.0).astype(np.float32)
    s0 = (g.standard_normal((H, S, S)) * 0.2).astype(np.float32)
    ns = np.zeros(T, np.uint8)
    ns[3] = 1
    s_fin, out = wkv7(r, w, k, v, a, b, s0, ns)
    doc = {"source": "numpy float64 restatement of the recurrence of rwkv7.py:200-220 (see gen_wkv7_golden.py)",
           "T": T, "H": H, "S": S,
           "inputs": {n: x.tolist() for n, x in (("r", r), ("w", w), ("k", k), ("v", v), ("a", a), ("b", b),
                                                 ("state", s0), ("new_starts", ns))},
           "state_out": s_fin.tolist(), "out": out.tolist()}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "wkv7_golden.json")
    with open(path, "w") as fh:
        json.dump(doc, fh)
    print("wrote", path)


if __name__ == "__main__":
    main()
