"""Genetar folder models on the GPU against the slow float64 implementation of tests/genetar_oracle.py.

Small random models (bf16-representable weights, so both operand modes load the same numbers) are written to a temporary
folder and opened through lmrs_b200.Transformer.open -- the entry point trace replay, forward, forward_argmax and
generate_greedy share.  float32 mode is held to 2e-4 of the logits' root mean square, bfloat16 mode to 4e-2."""
import numpy as np
import pytest

import genetar_oracle as G

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-4, "bfloat16": 4e-2}
SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


def mixed_cfg(**kw):
    """both mixers, grouped heads, a layer without feed-forward, one outside the value mixing, sizes that are no powers of two"""
    return G.make_config([
        G.attention_layer("attention_2", heads=6, kv_heads=2, dim=24, vdim=16, rot_dims=10, scaling=SCALING, scale=0.4, softcap=6.0),
        G.attention_layer("attention", heads=4, kv_heads=2, dim=16, vdim=16, scale=1.0, softcap=9.0, ff=0),
        G.attention_layer("attention", heads=2, kv_heads=2, dim=40, vdim=16, scale=0.7, softcap=4.0, v_mix=False, ff=40),
        G.attention_layer("attention_2", heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=16, scale=0.3, softcap=50.0, ff=72),
    ], **kw)


def open_model(gpu_lib, tmp_path, cfg, W, dtype, max_tokens=256, name="m"):
    return gpu_lib.Transformer.open(G.write_model(str(tmp_path / name), cfg, W), dtype=dtype, max_tokens=max_tokens)


def tokens_for(cfg, n, seed=0):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_logits_and_every_layer(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=1, qk_gain=2.0)
    toks = tokens_for(cfg, 45)
    want, outs = G.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype)
    assert m.args.model_type == gpu_lib.ModelType.GENETAR and m.args.vocab_size == cfg["vocab"] and m.args.n_layers == 4
    m.set_option("keep_layers", 1)
    got = m.forward_tokens(toks, 0, list(range(45)))
    lo = m.layer_outputs(45)
    for li in range(4):   # the first layer that differs names the broken mechanism
        assert G.rel_rms(lo[li], outs[li]) < TOL[dtype], f"residual stream after layer {li}"
    assert G.rel_rms(got, want) < TOL[dtype]
    assert m.kernel_launches() > 0
    m.close()


# each mechanism alone: a one-layer (or two-layer) model in which only that mechanism is not trivial
ALONE = {
    "unit_norm_attention": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False, scale=2.0, softcap=30.0)], bigram=None),
    "softcap_bites": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False, scale=6.0, softcap=1.5)], bigram=None),
    "no_softcap": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False, scale=1.0, softcap=None)], bigram=None),
    "rotary_partial": dict(layers=[G.attention_layer("attention_2", ff=0, v_mix=False, rot_dims=6, dim=16)], bigram=None),
    "rotary_full_scaled": dict(layers=[G.attention_layer("attention_2", ff=0, v_mix=False, rot_dims=16, dim=16, rot_base=50.0, scaling=SCALING)], bigram=None),
    "rotary_none": dict(layers=[G.attention_layer("attention_2", ff=0, v_mix=False, rot_dims=0)], bigram=None),
    "bigram": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False)], bigram=(1, 3, 5)),
    "bigram_large_multipliers": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False)], bigram=(97, 1000003, 65537)),
    "feed_forward": dict(layers=[G.attention_layer("attention", ff=56, v_mix=False)], bigram=None),
    "value_mixing": dict(layers=[G.attention_layer("attention", ff=0), G.attention_layer("attention_2", ff=0), G.attention_layer("attention", ff=0)], bigram=None),
    "value_mixing_starts_late": dict(layers=[G.attention_layer("attention", ff=0, v_mix=False), G.attention_layer("attention", ff=0), G.attention_layer("attention", ff=0)], bigram=None),
    "one_kv_head": dict(layers=[G.attention_layer("attention_2", heads=3, kv_heads=1, ff=0, v_mix=False)], bigram=None),
    "no_grouping": dict(layers=[G.attention_layer("attention", heads=3, kv_heads=3, ff=0, v_mix=False)], bigram=None),
    "many_heads_per_kv": dict(layers=[G.attention_layer("attention", heads=20, kv_heads=1, dim=8, vdim=8, ff=0, v_mix=False)], bigram=None),
    "wide_values": dict(layers=[G.attention_layer("attention", heads=2, kv_heads=1, dim=8, vdim=72, ff=0, v_mix=False)], bigram=None),
    "odd_width": dict(layers=[G.attention_layer("attention_2", dim=10, vdim=6, rot_dims=4, ff=23)], width=27, vocab=33),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(gpu_lib, tmp_path, name):
    kw = dict(ALONE[name])
    cfg = G.make_config(kw.pop("layers"), **kw)
    W = G.random_weights(cfg, seed=5, qk_gain=3.0)
    toks = tokens_for(cfg, 70, seed=2)   # crosses one key-tile border
    want, _ = G.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    got = m.forward_tokens(toks, 0, list(range(70)))
    assert G.rel_rms(got, want) < TOL["float32"]
    # and token by token through the decode step
    for i, t in enumerate(toks):
        lg = m.forward(t, i)
        if i in (0, 1, 63, 64, 65, 69):
            assert G.rel_rms(lg, want[i]) < TOL["float32"], f"decoded position {i}"
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_every_size_and_decoding_agree_with_the_whole_prompt(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=2, qk_gain=2.0)
    n = 150
    toks = tokens_for(cfg, n, seed=3)
    want, _ = G.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype)
    for cuts in ([n], [2] * 8 + [3, 61, 2, 64, 1, 1, 1, 1], [63, 1, 64, 2, 20], [1] * 6 + [129, 2, 13], [127, 23]):
        assert sum(cuts) == n
        at, rows = 0, []
        for c in cuts:   # the same handle again and again: what an earlier schedule left in the cache must not matter
            rows.append(m.forward_tokens(toks[at:at + c], at, list(range(c))))
            at += c
        assert G.rel_rms(np.concatenate(rows), want) < TOL[dtype], cuts
    # a long internal portion split by the library itself
    m.set_option("chunk_rows", 37)
    assert G.rel_rms(m.forward_tokens(toks, 0, list(range(n))), want) < TOL[dtype]
    m.close()


def test_wanted_rows_in_any_order(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=4)
    toks = tokens_for(cfg, 40)
    want, _ = G.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    idx = [39, 0, 17, 17, 5]
    assert G.rel_rms(m.forward_tokens(toks, 0, idx), want[idx]) < TOL["float32"]
    assert m.forward_tokens(toks, 0, []).shape == (0, cfg["vocab"])
    m.set_option("chunk_rows", 16)
    assert G.rel_rms(m.forward_tokens(toks, 0, idx), want[idx]) < TOL["float32"]
    m.close()


def test_a_far_key_that_dominates_is_found(gpu_lib, tmp_path):
    """One key far back gets a score that stands out.  Input dimension 0 is made private to two tokens (every other
    embedding is zero there); the query and key projections read it into one head dimension with a large weight.  The last
    token is one of the two, the other occurs once, far back: after the unit norm that key and the query's own are nearly
    parallel to the query, every other key is not.  The two tokens have different values, so leaving the far key out, or
    reading a neighbour instead, moves the logits by several percent.  Far key in the first tile, at tile borders and
    just before the query; in a prompt and in decoding."""
    layer = G.attention_layer("attention", heads=2, kv_heads=1, dim=16, vdim=16, ff=0, v_mix=False, scale=1.0, softcap=40.0)
    cfg = G.make_config([layer], width=16, vocab=50, bigram=None, logit_scale=1.0)
    W = G.random_weights(cfg, seed=7)
    a_tok, b_tok, n = 48, 49, 330
    W["embed"][:, 0] = 0.0
    W["embed"][[a_tok, b_tok], 0] = 4.0
    W["l0.mix.q"][:16, 0] = 0.0
    W["l0.mix.k"][:, 0] = 0.0
    W["l0.mix.q"][3, 0] = W["l0.mix.k"][3, 0] = 4.0
    eps = cfg["norm"]["eps"]
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32", max_tokens=400)
    for far in (0, 63, 64, 191, 192, n - 3):
        toks = [t if t < a_tok else 0 for t in tokens_for(cfg, n, seed=far)]
        toks[far], toks[n - 1] = a_tok, b_tok
        want, _ = G.forward(cfg, W, toks)
        # the slow implementation's own scores confirm that the case is what it claims to be
        h = G.rms(G.embed(toks, None, W, cfg), eps) * W["l0.norm1"]
        q = G.rms((h @ W["l0.mix.q"].T).reshape(n, 2, 16), eps)
        k = G.rms((h @ W["l0.mix.k"].T).reshape(n, 1, 16), eps)
        s = G.cap_scores(k[:, 0] @ q[n - 1, 0], 1.0, 40.0)
        assert s[far] >= np.sort(s)[-2] - 1e-9 and s[far] > np.sort(s)[-3] + 4.0
        toks2 = list(toks)
        toks2[far] = 0
        assert G.rel_rms(G.forward(cfg, W, toks2)[0][n - 1], want[n - 1]) > 100 * TOL["float32"]   # the check has teeth
        got = m.forward_tokens(toks, 0, [n - 1])
        assert G.rel_rms(got[0], want[n - 1]) < TOL["float32"], f"far key at {far} (prompt)"
        m.forward_tokens(toks[:n - 1], 0, [])
        assert G.rel_rms(m.forward(toks[n - 1], n - 1), want[n - 1]) < TOL["float32"], f"far key at {far} (decoded)"
    m.close()


def test_the_cache_is_reused_by_the_next_sequence(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=6)
    a, b = tokens_for(cfg, 90, seed=1), tokens_for(cfg, 33, seed=2)
    wa, _ = G.forward(cfg, W, a)
    wb, _ = G.forward(cfg, W, b)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    assert G.rel_rms(m.forward_tokens(a, 0, [89]), wa[[89]]) < TOL["float32"]
    # a shorter sequence over the same positions: nothing of `a` (keys beyond position 32, its last token) may show
    assert G.rel_rms(m.forward_tokens(b[:20], 0, [0, 19]), wb[[0, 19]]) < TOL["float32"]
    for i in range(20, 33):
        assert G.rel_rms(m.forward(b[i], i), wb[i]) < TOL["float32"]
    assert G.rel_rms(m.forward_tokens(a, 0, [0, 50]), wa[[0, 50]]) < TOL["float32"]
    m.close()


def test_first_tokens_and_a_prompt_of_one(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=8)
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32")
    for toks in ([7], [7, 7], [0, 1, 2]):
        want, _ = G.forward(cfg, W, toks)
        assert G.rel_rms(m.forward_tokens(toks, 0, list(range(len(toks)))), want) < TOL["float32"]
        assert G.rel_rms(m.forward(toks[0], 0), want[0]) < TOL["float32"]
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_greedy_generation_through_the_generate_loop(gpu_lib, tmp_path, dtype):
    cfg = mixed_cfg(logit_scale=3.0)
    W = G.random_weights(cfg, seed=9)
    prompt = tokens_for(cfg, 21, seed=4)
    n_new = 150   # decodes across two key-tile borders and through several key splits
    m = open_model(gpu_lib, tmp_path, cfg, W, dtype, max_tokens=21 + n_new)
    m.forward_tokens(prompt[:-1], 0, [])
    ids = m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist()
    assert len(ids) == n_new
    # replay the produced sequence through the slow implementation: every pick must be its argmax, or (bf16, f32 near-ties)
    # within a small margin of it
    seq = prompt + ids
    want, _ = G.forward(cfg, W, seq)
    margin = 1e-3 if dtype == "float32" else 0.15
    for i, t in enumerate(ids):
        row = want[len(prompt) - 1 + i]
        assert row[t] >= row.max() - margin * (row.max() - row.min()), f"generated token {i}"
    # forward_argmax is the same pick
    m.forward_tokens(prompt[:-1], 0, [])
    assert m.forward_argmax(prompt[-1], len(prompt) - 1) == ids[0]
    # decode steps replayed from CUDA graphs and launched one by one are the same arithmetic
    m.set_option("graphs", 0)
    m.forward_tokens(prompt[:-1], 0, [])
    assert m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist() == ids
    # ... and so are steps whose kernels are chained with programmatic dependent launch, replayed or not
    for graphs in (1, 0):
        m.set_option("graphs", graphs)
        m.set_option("pdl", 1)
        m.forward_tokens(prompt[:-1], 0, [])
        assert m.generate_greedy(prompt[-1], len(prompt) - 1, n_new).tolist() == ids
    with pytest.raises(gpu_lib.LmrsError):
        m.forward(1, 21 + n_new)   # beyond the cache
    m.close()


def test_tensor_core_products_equal_the_cuda_core_products(gpu_lib, tmp_path):
    """bf16 mode, shapes that are no multiples of the 128 x 128 x 64 tile: rows, outputs and K tails are masked or zero-filled"""
    cfg = G.make_config([
        G.attention_layer("attention_2", heads=5, kv_heads=5, dim=24, vdim=24, rot_dims=8, ff=200),
        G.attention_layer("attention", heads=6, kv_heads=2, dim=32, vdim=20, ff=136, v_mix=False),
    ], width=72, vocab=203)
    W = G.random_weights(cfg, seed=10)
    toks = tokens_for(cfg, 131)
    want, _ = G.forward(cfg, W, toks)
    m = open_model(gpu_lib, tmp_path, cfg, W, "bfloat16")
    a = m.forward_tokens(toks, 0, list(range(131)))
    m.set_option("tensor_cores", 0)
    b = m.forward_tokens(toks, 0, list(range(131)))
    assert G.rel_rms(a, b) < 5e-3 and not np.array_equal(a, b)   # different kernels, same numbers up to summation order
    assert G.rel_rms(a, want) < TOL["bfloat16"] and G.rel_rms(b, want) < TOL["bfloat16"]
    m.close()


def test_configuration_errors_are_reported(gpu_lib, tmp_path):
    cfg = mixed_cfg()
    W = G.random_weights(cfg)
    bad = dict(cfg, architecture="NoSuchModel")
    with pytest.raises(gpu_lib.LmrsError, match="unknown architecture"):
        gpu_lib.Transformer.open(G.write_model(str(tmp_path / "a"), bad, W))
    W2 = {k: v for k, v in W.items() if k != "l2.mix.o"}
    with pytest.raises(gpu_lib.LmrsError, match="l2.mix.o"):
        gpu_lib.Transformer.open(G.write_model(str(tmp_path / "b"), cfg, W2))
    W3 = dict(W, head=W["head"][:-1])
    with pytest.raises(gpu_lib.LmrsError, match="head"):
        gpu_lib.Transformer.open(G.write_model(str(tmp_path / "c"), cfg, W3))
    m = open_model(gpu_lib, tmp_path, cfg, W, "float32", max_tokens=16)
    with pytest.raises(gpu_lib.LmrsError):
        m.forward_tokens([1] * 17, 0, [])
    with pytest.raises(gpu_lib.LmrsError, match="token"):
        m.forward_tokens([cfg["vocab"]], 0, [])
    with pytest.raises(gpu_lib.LmrsError):
        m.get_embeddings([1])
    m.close()


def test_the_command_line_generates_from_a_folder(gpu_lib, tmp_path):
    """lm.rs_b200/examples/generate on a model folder prints the ids that generate_greedy picks"""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.check_call(["make", "-C", os.path.join(root, "lm.rs_b200"), "-s", "examples"])
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=11)
    d = G.write_model(str(tmp_path / "cli"), cfg, W)
    prompt = [3, 9, 27, 20]
    env = dict(os.environ, GENERATE_DTYPE="float32")
    r = subprocess.run([os.path.join(root, "lm.rs_b200", "examples", "generate"), d, "10"] + [str(t) for t in prompt],
                       capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    m = gpu_lib.Transformer.open(d, dtype="float32", max_tokens=32)
    m.forward_tokens(prompt[:-1], 0, [])
    assert [int(x) for x in r.stdout.split()] == m.generate_greedy(prompt[-1], 3, 10).tolist()
    m.close()


def test_trace_replay_writes_the_logits_asked_for(gpu_lib, tmp_path):
    """bin/trace_run: a prompt in portions, then single tokens, then a second request over the same cache"""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = mixed_cfg()
    W = G.random_weights(cfg, seed=12)
    d = G.write_model(str(tmp_path / "tr"), cfg, W)
    a, b = tokens_for(cfg, 75, seed=5), tokens_for(cfg, 9, seed=6)
    wa, _ = G.forward(cfg, W, a)
    wb, _ = G.forward(cfg, W, b)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:73], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[73:74], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[74:75], "want": [0]}], "end": ["x"]},
             {"step": 4, "entries": [{"id": "y", "tokens": b, "want": [8, 2]}], "end": ["y"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "80"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done %d" % i for i in range(5)]
    assert not (out / "1.f32").exists()
    V = cfg["vocab"]
    for step, want in ((0, wa[[0, 65]]), (2, wa[[73]]), (3, wa[[74]]), (4, wb[[8, 2]])):
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, V)
        assert G.rel_rms(got, want) < TOL["float32"], f"step {step}"


def test_lmrs_files_open_by_path_and_take_token_steps(gpu_lib, lf, tmp_path):
    """the path-based entry point serves the LMRS models too: forward_tokens on them is a run of decode steps"""
    buf = lf.write_synthetic(lf.model_args("tiny-llama", 1))
    path = tmp_path / "tiny.lmrs"
    buf.tofile(path)
    m = gpu_lib.Transformer.open(str(path))
    ref, _ = gpu_lib.Transformer.new(buf)
    toks = [3, 1, 4, 1, 5, 9]
    got = m.forward_tokens(toks, 0, [5, 2])
    rows = [ref.forward(t, i).copy() for i, t in enumerate(toks)]
    assert np.array_equal(got[0], rows[5]) and np.array_equal(got[1], rows[2])
    with pytest.raises(gpu_lib.LmrsError):
        gpu_lib.Transformer.open(str(path), dtype="float32")
    m.close(); ref.close()
