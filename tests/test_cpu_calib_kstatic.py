"""The oracle's K-static fit against the formula the synthetic tables are built with
(synth.make_tables: sigma = per-dim std of the projected sample, ts = 16 / sqrt(sum 0.528756
(0.935 sigma)^2 + 0.464545 sigma^2), centroid rows {0, -cb, cb, cb})."""
import numpy as np

from bonsai_mojo_1bit_optimization_t4_cuda_b200 import synth


def test_kstatic_matches_the_table_generator(oracle):
    rng = np.random.default_rng(21)
    k, v = synth.make_kv(rng, 96)
    d_k = synth.xorshift_signs(3, "k")
    rot = synth.project(k.reshape(-1, 256), d_k, synth.random_rotors(rng))
    cents, ts, sigma = oracle.cal_kstatic(rot)
    sig = rot.astype(np.float64).std(axis=0)
    psum = 0.528756 * (0.9350 * sig) ** 2 + 0.464545 * sig ** 2
    ts_want = 16.0 / np.sqrt(psum.sum())
    assert np.allclose(sigma, sig, rtol=2e-5, atol=1e-7)
    assert abs(ts - ts_want) <= 2e-5 * ts_want
    cb = 0.9350 * sig * ts_want
    assert np.allclose(cents[0], 0) and np.allclose(cents[1], -cb, rtol=5e-5) and np.allclose(cents[2], cb, rtol=5e-5)
    assert np.array_equal(cents[2], cents[3]) and np.array_equal(cents[1], -cents[2])
