"""Plain, slow float64 implementation of the Tudatar architecture: test infrastructure only.

One function per mechanism, written from the equations below in numpy; it shares no code with the library.

    layer          x <- x + N1b(mixer(N1(x)));  x <- x + N2b(ff(N2(x)))          (the second line only with a feed-forward)
    N(x)           tanh(alpha * x) * w + b          (no mean, no variance)
    rms(x)         x / sqrt(mean(x^2) + eps)
    mixer D        gated delta rule with one decay per key channel (delta_*):
                     q, k, v <- silu(causal_conv(W h));  q, k <- unit vectors per head;  q <- q / sqrt(dim)
                     beta = sigmoid(W_b h);  g = exp(-exp(A_log) * softplus(W_a2 W_a1 h + dt_bias))
                     S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                     out = W_o (rms(o) * w_norm * sigmoid(W_g2 W_g1 h))
    mixer L        attention through a latent (latent_*):
                     cq = rms(W_dq h) * w;  q = W_uq cq = per head [plain | rotated]
                     [c_raw | kr] = W_dkv h;  c = rms(c_raw) * w;  k_h = [W_uk c | rot(kr)],  v_h = W_uv c
                     rotation pairs dimensions (2i, 2i+1); frequencies rescaled by a ramp between two wavelengths, cos and sin
                     multiplied by 0.1 ln(factor) + 1;  causal softmax(scale * q.k)
    mixer W        windowed attention (window_*): biases on q, k, v;  q, k <- rms over the WHOLE projection * w;
                     v <- unit rms per head;  s = scale * q.k - r1_h ln(1 + r2_h (i - j)),  0 <= i - j < window;  softmax
    ff             z = W_r h;  s = sigmoid(z);  the `top` largest of s + correction are chosen;
                     weights = s_chosen / (sum s_chosen + 1e-20) * router_scale;  sum of weight * expert(h)
                     expert(h) = W_down (silu(W_gate h) * (W_up h))
    logits         logit_scale * W_head N_final(x)

StepOracle carries the state (recurrent matrices, convolution tails, key/value lists) from call to call, so the
whole-sequence functions and the incremental form check each other.  make_config / random_weights / write_model build
small random model folders (config.json + model.safetensors with bf16 tensors).
"""
import json
import math
import os
import struct

import numpy as np


# ---- number formats -----------------------------------------------------------------------------------------------------
def to_bf16_bits(a):
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_round(a):
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


# ---- small functions --------------------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def tanh_norm(x, W, name):
    """tanh(alpha x) w + b with the scalar `name.alpha` and the vector `name.b`"""
    return np.tanh(float(W[name + ".alpha"]) * x) * W[name] + W[name + ".b"]


# ---- rotation with rescaled frequencies -----------------------------------------------------------------------------------------
def rot_freqs(rot):
    """(frequencies [dims/2], multiplier of cos and sin)"""
    d, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / d) for i in range(d // 2)], np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def where(turns):   # the (fractional) pair index whose wavelength makes `turns` turns over the original length
        return d * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), d - 1)
    ramp = np.clip((np.arange(d // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, positions, rot):
    """x [..., T, n >= dims]: the first dims entries rotated pairwise (2i, 2i+1) by positions * f_i"""
    f, mult = rot_freqs(rot)
    d = rot["dims"]
    ang = np.asarray(positions, np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang) * mult, np.sin(ang) * mult
    out = x.copy()
    u, v = x[..., 0:d:2], x[..., 1:d:2]
    out[..., 0:d:2] = u * c - v * s
    out[..., 1:d:2] = v * c + u * s
    return out


# ---- mixer D: gated delta rule ------------------------------------------------------------------------------------------------
def causal_conv(x, w, tail):
    """x [T, C], w [C, taps] (last column multiplies the current token), tail [taps-1, C] = the inputs before x.
    Returns (y [T, C], new tail)."""
    taps = w.shape[1]
    full = np.concatenate([tail, x], 0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += full[j:j + x.shape[0]] * w[:, j][None, :]
    return y, full[full.shape[0] - (taps - 1):].copy()


def unit(x):
    return x / np.sqrt(np.sum(x * x, -1, keepdims=True) + 1e-6)


def delta_scan(q, k, v, g, beta, S):
    """q, k, g [T, H, dk]; v [T, H, dv]; beta [T, H]; S [H, dk, dv] is updated in place. Returns o [T, H, dv]."""
    T, H, dv = v.shape
    o = np.zeros((T, H, dv))
    for t in range(T):
        for h in range(H):
            S[h] *= g[t, h][:, None]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] += np.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o


def delta_mixer(h, W, p, m, eps, state):
    """state: dict with 'S' [H, dk, dv] and 'tail_q', 'tail_k', 'tail_v' (or empty at the start of a sequence)"""
    T = h.shape[0]
    H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    if "S" not in state:
        state["S"] = np.zeros((H, dk, dv))
        for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
            state["tail_" + n] = np.zeros((taps - 1, c))
    out = {}
    for n in ("q", "k", "v"):
        y, state["tail_" + n] = causal_conv(h @ W[p + n].T, W[p + n + ".conv"], state["tail_" + n])
        out[n] = silu(y)
    rep = H // G
    q = np.repeat(unit(out["q"].reshape(T, G, dk)) * dk ** -0.5, rep, axis=1)
    k = np.repeat(unit(out["k"].reshape(T, G, dk)), rep, axis=1)
    v = out["v"].reshape(T, H, dv)
    beta = sigmoid(h @ W[p + "b"].T)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, dk))
    o = delta_scan(q, k, v, g, beta, state["S"])
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, dv)
    o = rms(o, eps) * W[p + "norm"][None, None, :] * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---- softmax attention over explicit key/value lists ------------------------------------------------------------------------------
def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def latent_mixer(h, W, p, m, eps, state, pos0):
    """state: 'c' [n, kv_rank] and 'kr' [n, rot_dim] of the tokens so far (kr already rotated)"""
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(pos0, pos0 + T)
    cq = rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate_pairs(q[..., dn:].transpose(1, 0, 2), pos, m["rot"]).transpose(1, 0, 2)
    ckr = h @ W[p + "dkv"].T
    c = rms(ckr[:, :rk], eps) * W[p + "dkv.norm"]
    kr = rotate_pairs(ckr[:, rk:], pos, m["rot"])
    state["c"] = np.concatenate([state["c"], c], 0) if "c" in state else c
    state["kr"] = np.concatenate([state["kr"], kr], 0) if "kr" in state else kr
    C, KR = state["c"], state["kr"]
    n = C.shape[0]
    kn = (C @ W[p + "uk"].T).reshape(n, H, dn)
    vv = (C @ W[p + "uv"].T).reshape(n, H, dv)
    s = (np.einsum("thd,nhd->htn", qn, kn) + np.einsum("thd,nd->htn", qr, KR)) * m["scale"]
    vis = np.arange(n)[None, :] <= pos[:, None]
    a = softmax_rows(s, vis[None])
    o = np.einsum("htn,nhd->thd", a, vv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def window_mixer(h, W, p, m, eps, state, pos0):
    """state: 'k' [n, G, dk], 'v' [n, G, dv] of the tokens so far (after their norms)"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(pos0, pos0 + T)
    q = rms(h @ W[p + "q"].T + W[p + "q.b"], eps) * W[p + "q.norm"]
    k = rms(h @ W[p + "k"].T + W[p + "k.b"], eps) * W[p + "k.norm"]
    v = rms((h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv), eps)
    k = k.reshape(T, G, dk)
    state["k"] = np.concatenate([state["k"], k], 0) if "k" in state else k
    state["v"] = np.concatenate([state["v"], v], 0) if "v" in state else v
    K, V = np.repeat(state["k"], H // G, 1), np.repeat(state["v"], H // G, 1)
    n = K.shape[0]
    dist = pos[:, None] - np.arange(n)[None, :]
    vis = (dist >= 0) & (dist < m["mask"]["size"])
    far = np.log1p(W[p + "r2"][:, None, None] * np.maximum(dist, 0)[None]) * W[p + "r1"][:, None, None]
    s = np.einsum("thd,nhd->htn", q.reshape(T, H, dk), K) * m["scale"] - far
    a = softmax_rows(s, vis[None])
    o = np.einsum("htn,nhd->thd", a, V)
    return o.reshape(T, H * dv) @ W[p + "o"].T


# ---- feed-forward: routed experts -----------------------------------------------------------------------------------------------------
CHOICE_GAPS = []   # per route() call: the smallest distance between the last chosen and the first rejected expert


def route(h, W, p, r):
    """(chosen experts [T, top], their weights [T, top])"""
    s = sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    order = np.argsort(-choice, axis=-1, kind="stable")
    idx = order[:, :r["top"]]
    if r["top"] < choice.shape[-1]:
        ranked = np.take_along_axis(choice, order, -1)
        CHOICE_GAPS.append(float((ranked[:, r["top"] - 1] - ranked[:, r["top"]]).min()))
    w = np.take_along_axis(s, idx, -1)
    return idx, w / (w.sum(-1, keepdims=True) + 1e-20) * r["scale"]


def expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_ff(h, W, p, f):
    idx, w = route(h, W, p, f["router"])
    y = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t]):
            y[t] += w[t, j] * expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    return y


# ---- the model ----------------------------------------------------------------------------------------------------------------------------
class StepOracle:
    """Feeds tokens in portions; keeps every layer's state between calls."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, {k: np.asarray(v, np.float64) for k, v in W.items()}
        self.state = [dict() for _ in cfg["layers"]]
        self.pos = 0

    def step(self, tokens):
        """-> (logits [T, vocab], residual stream after every layer [layers, T, width])"""
        cfg, W, eps = self.cfg, self.W, self.cfg["norm"]["eps"]
        x = W["embed"][np.asarray(tokens, np.int64)].copy()
        outs = []
        for i, L in enumerate(cfg["layers"]):
            p, m = f"l{i}.", L["mixer"]
            h = tanh_norm(x, W, p + "norm1")
            if L["type"] == "channel_delta":
                y = delta_mixer(h, W, p + "mix.", m, eps, self.state[i])
            elif L["type"] == "latent_attention":
                y = latent_mixer(h, W, p + "mix.", m, eps, self.state[i], self.pos)
            elif L["type"] == "attention":
                y = window_mixer(h, W, p + "mix.", m, eps, self.state[i], self.pos)
            else:
                raise ValueError(L["type"])
            x = x + tanh_norm(y, W, p + "norm1b")
            if L.get("mlp"):
                x = x + tanh_norm(routed_ff(tanh_norm(x, W, p + "norm2"), W, p + "mlp.", L["mlp"]), W, p + "norm2b")
            outs.append(x.copy())
        self.pos += len(tokens)
        logits = tanh_norm(x, W, "final.norm") @ W["head"].T * cfg.get("logit_scale", 1.0)
        return logits, np.stack(outs)


def forward(cfg, W, tokens):
    return StepOracle(cfg, W).step(tokens)


def clear_choices(cfg, W, tokens, gap):
    """True when no routing decision of this run is closer than `gap` (a test in reduced precision must not rest on one)"""
    del CHOICE_GAPS[:]
    forward(cfg, W, tokens)
    return all(g > gap for g in CHOICE_GAPS)


def rel_rms(got, want):
    """root mean square of the difference over that of `want`, means over the last axis taken off"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float(np.sqrt(np.mean(d * d)) / (np.sqrt(np.mean(w * w)) + 1e-30))


# ---- small random models -----------------------------------------------------------------------------------------------------------------
def moe(experts=6, top=2, ff=24, scale=1.25):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def delta_layer(heads=4, kv_heads=2, dim=12, vdim=20, conv=4, mlp="default"):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": moe() if mlp == "default" else mlp}


def latent_layer(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=40, scale=0.3, base=100.0, scaling="default", mlp="default"):
    rot = {"base": base, "dims": rot_dim}
    if scaling == "default":
        scaling = {"factor": 4.0, "fast": 8.0, "slow": 1.0, "original": 32}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                    "q_rank": q_rank, "scale": scale, "rot": rot},
            "mlp": moe() if mlp == "default" else mlp}


def window_layer(heads=4, kv_heads=2, dim=12, vdim=20, window=9, scale=0.5, mlp="default"):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "mask": {"size": window}},
            "mlp": moe() if mlp == "default" else mlp}


def make_config(layers, width=40, vocab=70, eps=1e-5, logit_scale=0.5):
    return {"architecture": "Tudatar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}


def tensor_table(cfg):
    """[(name, shape, kind)]; kind: matrix | table | gain | shift | alpha | conv | small | rate | zero"""
    w = cfg["width"]

    def norm(n, size):
        return [(n, (size,), "gain"), (n + ".b", (size,), "shift"), (n + ".alpha", (), "alpha")]
    out = [("embed", (cfg["vocab"], w), "table")]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm2", "norm1b", "norm2b"):
            out += norm(p + n, w)
        q = p + "mix."
        if L["type"] == "channel_delta":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            ra, rg = m.get("a_rank", 6), m.get("g_rank", 10)
            out += [(q + "q", (G * dk, w), "matrix"), (q + "q.conv", (G * dk, m["conv"]), "conv"), (q + "k", (G * dk, w), "matrix"),
                    (q + "k.conv", (G * dk, m["conv"]), "conv"), (q + "v", (H * dv, w), "matrix"), (q + "v.conv", (H * dv, m["conv"]), "conv"),
                    (q + "b", (H, w), "matrix"), (q + "A_log", (H,), "rate"), (q + "norm", (dv,), "gain"),
                    (q + "a1", (ra, w), "matrix"), (q + "a2", (H * dk, ra), "matrix"), (q + "dt_bias", (H * dk,), "shift"),
                    (q + "g1", (rg, w), "matrix"), (q + "g2", (H * dv, rg), "matrix"), (q + "o", (w, H * dv), "matrix")]
        elif L["type"] == "latent_attention":
            H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out += [(q + "dq", (rq, w), "matrix"), (q + "dq.norm", (rq,), "gain"), (q + "uq", (H * (dn + dr), rq), "matrix"),
                    (q + "dkv", (rk + dr, w), "matrix"), (q + "dkv.norm", (rk,), "gain"), (q + "uk", (H * dn, rk), "matrix"),
                    (q + "uv", (H * dv, rk), "matrix"), (q + "o", (w, H * dv), "matrix")]
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out += [(q + "q", (H * dk, w), "matrix"), (q + "q.b", (H * dk,), "shift"), (q + "k", (G * dk, w), "matrix"),
                    (q + "k.b", (G * dk,), "shift"), (q + "v", (G * dv, w), "matrix"), (q + "v.b", (G * dv,), "shift"),
                    (q + "q.norm", (H * dk,), "gain"), (q + "k.norm", (G * dk,), "gain"), (q + "r1", (H,), "small"),
                    (q + "r2", (H,), "small"), (q + "o", (w, H * dv), "matrix")]
        if L.get("mlp"):
            f = L["mlp"]
            out += [(p + "mlp.router", (f["router"]["experts"], w), "matrix"), (p + "mlp.correction", (f["router"]["experts"],), "zero")]
            for e in range(f["router"]["experts"]):
                out += [(f"{p}mlp.e{e}.gate", (f["expert"]["ff"], w), "matrix"), (f"{p}mlp.e{e}.up", (f["expert"]["ff"], w), "matrix"),
                        (f"{p}mlp.e{e}.down", (w, f["expert"]["ff"]), "matrix")]
    return out + norm("final.norm", w) + [("head", (cfg["vocab"], w), "matrix")]


def random_weights(cfg, seed=0, gain=1.0):
    """bf16-representable float64 weights"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape, kind in tensor_table(cfg):
        n = int(np.prod(shape)) if shape else 1
        if kind == "matrix":
            a = rng.standard_normal(n) * gain / math.sqrt(shape[-1])
            if name.endswith("router"):
                a *= 3.0
        elif kind == "table":
            a = rng.standard_normal(n)
        elif kind == "gain":
            a = 1.0 + 0.2 * rng.standard_normal(n)
        elif kind == "shift":
            a = 0.2 * rng.standard_normal(n)
        elif kind == "alpha":
            a = np.array([0.6 + 0.3 * rng.random()])
        elif kind == "conv":
            a = rng.standard_normal(n) * 0.6
        elif kind == "small":
            a = 0.1 + 0.5 * rng.random(n)
        elif kind == "rate":
            a = -1.0 + rng.standard_normal(n)
        else:
            a = 0.3 * rng.standard_normal(n)
        W[name] = bf16_round(a).reshape(shape)
    return W


def write_model(folder, cfg, W):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, a in W.items():
        b = to_bf16_bits(np.asarray(a, np.float32)).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b)
    return folder
