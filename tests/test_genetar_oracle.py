"""The slow Genetar implementation of tests/genetar_oracle.py against itself and against hand-made cases (no GPU):
whole-sequence arithmetic == incremental arithmetic over explicit K/V lists, and each mechanism on inputs whose answer
is known in closed form.  The model-folder writer is checked against a byte-level read of its own file."""
import json
import math
import os
import struct

import numpy as np
import pytest

import genetar_oracle as G


def small_cfg():
    return G.make_config([
        G.attention_layer("attention_2", heads=4, kv_heads=2, dim=12, vdim=8, rot_dims=6, scaling={"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}),
        G.attention_layer("attention", heads=6, kv_heads=2, dim=8, vdim=8, v_mix=True, ff=0),
        G.attention_layer("attention", heads=2, kv_heads=2, dim=8, vdim=8, v_mix=False),
        G.attention_layer("attention_2", heads=4, kv_heads=2, dim=16, vdim=8, rot_dims=16, v_mix=True),
    ], width=24, vocab=37)


def test_whole_sequence_equals_portions_and_single_tokens():
    cfg = small_cfg()
    W = G.random_weights(cfg, seed=3)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 19).tolist()
    whole, outs = G.forward(cfg, W, toks)
    assert outs.shape == (4, 19, 24)
    for cuts in ([19], [1] * 19, [2, 3, 5, 7, 2], [18, 1]):
        inc, got, at = G.IncrementalOracle(cfg, W), [], 0
        for c in cuts:
            got.append(inc.step(toks[at:at + c]))
            at += c
        assert np.allclose(np.concatenate(got), whole, rtol=0, atol=1e-9)


def test_bigram_rows():
    assert G.bigram_rows([4, 9, 9], None, 11, 7, 3).tolist() == [11, (4 * 7 + 9 * 3) % 11, (9 * 7 + 9 * 3) % 11]
    assert G.bigram_rows([5], 2, 11, 7, 3).tolist() == [(2 * 7 + 5 * 3) % 11]
    assert G.bigram_rows([0, 0], None, 1, 3, 5).tolist() == [1, 0]   # one bucket: every pair hashes to row 0


def test_rms_has_eps_inside_the_root():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(G.rms(x, 0.5), x / math.sqrt(12.5 + 0.5))
    assert np.allclose(G.rms(np.zeros((1, 4)), 1e-6), 0.0)


def test_rotary_pairs_first_dims_only_and_keeps_norm():
    rot = {"base": 100.0, "dims": 4}
    z = np.arange(1.0, 7.0).reshape(1, 1, 6)
    r = G.rotary(z, [3], rot)
    f = G.rotary_freqs(rot)
    assert np.allclose(f, [1.0, 100.0 ** -0.5])
    a0, a1 = 3 * f[0], 3 * f[1]
    assert np.allclose(r[0, 0], [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                 3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5, 6])
    assert np.allclose(G.rotary(z, [0], rot), z)


def test_rotary_frequency_scaling_bands():
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100}
    rot = {"base": 10000.0, "dims": 16, "scaling": sc}
    plain = G.rotary_freqs({"base": 10000.0, "dims": 16})
    f = G.rotary_freqs(rot)
    wl = 2 * math.pi / plain
    short, long_ = wl < 100 / 4.0, wl > 100 / 1.0
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert np.allclose(f[short], plain[short]) and np.allclose(f[long_], plain[long_] / 4.0)
    mid = ~short & ~long_
    assert ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 4.0)).all()


def test_softcap_and_causal_softmax():
    assert np.allclose(G.cap_scores(np.array([100.0, -100.0, 0.1]), 0.5, 5.0), [5 * math.tanh(10), -5 * math.tanh(10), 5 * math.tanh(0.01)])
    assert np.allclose(G.cap_scores(np.array([3.0]), 2.0, None), [6.0])
    q = np.zeros((2, 2, 3))
    K = np.zeros((2, 1, 3))
    V = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    o = G.attend(q, K, V, [0, 1], 1.0, 10.0)
    assert np.allclose(o[0], [[1, 0], [1, 0]]) and np.allclose(o[1], [[0.5, 0.5], [0.5, 0.5]])


def test_value_mixing_and_grouped_heads():
    assert np.allclose(G.mix_values(np.array([2.0]), np.array([10.0]), 0.25), [4.0])
    # query head h reads KV head h // (H / G): make the two KV heads return different values
    q = np.ones((1, 4, 2))
    K = np.ones((1, 2, 2))
    V = np.array([[[1.0], [2.0]]])
    assert np.allclose(G.attend(q, K, V, [0], 1.0, None)[0, :, 0], [1, 1, 2, 2])


def test_written_folder_reads_back(tmp_path):
    cfg = small_cfg()
    W = G.random_weights(cfg, seed=1)
    d = G.write_model(str(tmp_path / "m"), cfg, W)
    assert json.load(open(os.path.join(d, "config.json")))["architecture"] == "Genetar"
    raw = open(os.path.join(d, "model.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    assert set(hdr) == set(G.tensor_shapes(cfg))
    lo, hi = hdr["l1.mix.q"]["data_offsets"]
    back = (np.frombuffer(raw[8 + n + lo:8 + n + hi], np.uint16).astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(back.reshape(hdr["l1.mix.q"]["shape"]), W["l1.mix.q"].astype(np.float32))
    assert hdr["l0.mix.vmix"]["shape"] == []


@pytest.mark.skipif(os.path.exists("/dev/nvidia0"), reason="GPU present: the no-GPU failure path cannot be exercised")
def test_folder_models_fail_loudly_without_a_gpu(gpu_lib, tmp_path):
    cfg = small_cfg()
    d = G.write_model(str(tmp_path / "m"), cfg, G.random_weights(cfg))
    with pytest.raises(gpu_lib.LmrsError, match="no CUDA device|no CPU fallback"):
        gpu_lib.Transformer.open(d)
