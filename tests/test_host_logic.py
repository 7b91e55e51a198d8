"""Host-side logic that needs no GPU: pair folding of scattered fitness
vectors, the epoch/thread mapping, and the calibration scheme itself (the
fp64 candidates plus flip bitmaps reproduce the host libm bit for bit)."""
import os
import subprocess

import pytest
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_epoch_thread_sign_matches_oracle(oracle):
    from hyperscalees_b200 import noiser
    for epoch, tid, reuse in [(0, 0, 0), (7, 5, 0), (7, 4, 2), (9, 13, 3), (-3, 2, 2)]:
        assert noiser.epoch_thread_sign(noiser.IterInfo(epoch, tid), reuse) == oracle.epoch_thread_sign(epoch, tid, reuse)


def test_dense_fitness_scatter():
    from hyperscalees_b200 import noiser
    infos = [noiser.IterInfo(0, 5), noiser.IterInfo(0, 2), noiser.IterInfo(4, 9), noiser.IterInfo(0, 5)]
    d = noiser._dense_fitness(np.array([1.0, 2.0, 3.0, 0.5], np.float32), infos, 2)
    assert set(d) == {0, 2}
    lo, vec = d[0]
    assert lo == 2 and vec.tolist() == [2.0, 0.0, 0.0, 1.5]
    lo, vec = d[2]
    assert lo == 8 and vec.tolist() == [0.0, 3.0]


def test_solver_constructors_follow_reference_defaults():
    from hyperscalees_b200 import noiser
    s = noiser.Solver.adamw(0.01)
    assert (s.beta1, s.beta2, s.eps, s.weight_decay) == (0.9, 0.999, 1e-8, 1e-4)
    assert noiser.Solver.adam(0.01).weight_decay == 0.0


def test_calibration_scheme_reproduces_host_libm(tmp_path):
    """Compiles the host/device-portable RNG header for the CPU and checks that
    candidate + flip bitmap equals logf/cosf-based Box-Muller on 2M normals."""
    src = tmp_path / "calib_check.cpp"
    src.write_text(r'''
#include "hyperscalees_b200/csrc/rng.cuh"
#include "hyperscalees_b200/csrc/calib.hpp"
#include <stdio.h>
using namespace hses;
int main() {
    std::vector<double> tab(128); build_log_table(tab.data());
    std::vector<uint32_t> b(kUnits), c(kUnits);
    auto fill = [&](int which) {
        for (uint32_t i = which == 0 ? 1 : 0; i < kUnits; ++i) {
            Rounded r = which == 0 ? round_candidate(log_candidate(i, (const double2*)tab.data()))
                                   : round_candidate(cos_candidate(fmul(kTauF, (float)i * 5.9604644775390625e-08f)));
            b[i] = r.bits; c[i] = r.dist | ((r.alt < r.bits) ? 0x80000000u : 0u);
        }
    };
    CalibResult L, Cc;
    fill(0); calibrate(b.data(), c.data(), 1u, host_logf_u24, L);
    fill(1); calibrate(b.data(), c.data(), 0u, host_cosf_u24, Cc);
    if (!L.error.empty() || !Cc.error.empty()) { printf("ERR %s %s\n", L.error.c_str(), Cc.error.c_str()); return 1; }
    LibmCal cal{(const double2*)tab.data(), L.flip.data(), Cc.flip.data(), L.delta, Cc.delta, logf(1e-9f)};
    uint64_t s = 0x8aed0390bd5bae2ull | 1, s2 = s; long bad = 0;
    for (int n = 0; n < 2000000; ++n) {
        float z = next_normal(s, cal);
        uint64_t x1 = xs64_step(s2), x2 = xs64_step(x1); s2 = x2;
        float u1 = fmaxf((float)(x1 >> 40) / 16777216.0f, 1e-9f), u2 = (float)(x2 >> 40) / 16777216.0f;
        float ref = sqrtf(-2.0f * logf(u1)) * cosf(6.2831855f * u2);
        if (f2u(z) != f2u(ref)) bad++;
    }
    printf("OK flips %lu %lu bad %ld\n", (unsigned long)L.n_flips, (unsigned long)Cc.n_flips, bad);
    return bad != 0;
}
''')
    exe = tmp_path / "calib_check"
    # fma() must be the hardware instruction: the software fallback of libm is two orders of
    # magnitude slower over 2 * 2^24 candidates
    try:
        with open("/proc/cpuinfo") as fh:
            has_fma = any(" fma " in line + " " for line in fh if line.startswith("flags"))
    except OSError:
        has_fma = False
    if not has_fma:
        pytest.skip("this CPU has no FMA instruction")
    subprocess.run(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-mfma", "-pthread", "-I", ROOT,
                    str(src), "-o", str(exe), "-lm"], check=True, env={k: v for k, v in os.environ.items() if k not in ("CC", "CXX")})
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.startswith("OK")
