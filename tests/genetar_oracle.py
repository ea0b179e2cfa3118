"""Plain, slow float64 implementation of the Genetar architecture: test infrastructure only.

One function per mechanism, written from the equations below in numpy; it shares no code with the library.

    embedding      x_t = E[tok_t] + B[r_t],   r_t = (tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets,  r_0 = buckets
    block          h = rms(x) * w_norm1;   x <- x + ls1 * mixer(h) + ls2 * ff(h)
    rms(x)         x / sqrt(mean(x^2) + eps)
    mixer A        q, k <- rms(q), rms(k) per head (no weight);  no positions
    mixer B        first `dims` dimensions of q, k rotated: (u_i, u_{i+dims/2}) by angle p * f_i, f_i = base^(-2i/dims),
                   optionally rescaled by wavelength (long: f / factor, short: f, between: linear blend);
                   head output times sigmoid(W_g h)
    scores         s = scale * q.k;  s <- cap * tanh(s / cap);  causal softmax
    value mixing   v <- (1 - lam) v + lam v_first in every mixing layer after the first one; the mixed v is what is cached
    ff             W_down (silu(W_gate h) * (W_up h))
    logits         logit_scale * W_head (rms(x) * w_final)

Also: make_config / random_weights / write_model build a small random model folder (config.json + model.safetensors with
bf16 tensors), and IncrementalOracle runs the same arithmetic one token at a time over explicit K/V lists, so that the
whole-sequence functions and the cached form check each other.
"""
import json
import math
import os
import struct

import numpy as np


# ---- number formats -----------------------------------------------------------------------------------------------------
def to_bf16_bits(a):
    """float -> bfloat16 bit patterns (round to nearest even)"""
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_round(a):
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


# ---- mechanisms -----------------------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def bigram_rows(tokens, prev_token, buckets, mul_prev, mul_cur):
    """row of the bigram table for every token; prev_token = None at the start of a sequence"""
    rows, prev = [], prev_token
    for t in tokens:
        rows.append(buckets if prev is None else (int(prev) * mul_prev + int(t) * mul_cur) % buckets)
        prev = t
    return np.array(rows, np.int64)


def embed(tokens, prev_token, W, cfg):
    x = W["embed"][np.asarray(tokens, np.int64)].copy()
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][bigram_rows(tokens, prev_token, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


def rotary_freqs(rot):
    d = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / d) for i in range(d // 2)], np.float64)
    sc = rot.get("scaling")
    if sc:
        out = f.copy()
        for i, fi in enumerate(f):
            wl = 2.0 * math.pi / fi
            if wl < sc["original"] / sc["high"]:
                out[i] = fi
            elif wl > sc["original"] / sc["low"]:
                out[i] = fi / sc["factor"]
            else:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
        f = out
    return f


def rotary(z, positions, rot):
    """z [T][heads][dim]; rotates the first rot['dims'] dimensions, pairs (i, i + dims/2)"""
    d = rot["dims"]
    if d == 0:
        return z
    f = rotary_freqs(rot)
    ang = np.asarray(positions, np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, w = z[..., : d // 2], z[..., d // 2: d]
    return np.concatenate([u * c - w * s, w * c + u * s, z[..., d:]], axis=-1)


def cap_scores(s, scale, softcap):
    s = s * scale
    return softcap * np.tanh(s / softcap) if softcap else s


def attend(q, K, V, q_positions, scale, softcap):
    """q [T][H][dk]; K [S][G][dk], V [S][G][dv] hold keys 0..S-1; row t sees keys j <= q_positions[t]"""
    T, H, _ = q.shape
    G = K.shape[1]
    out = np.zeros((T, H, V.shape[2]))
    for t in range(T):
        n = int(q_positions[t]) + 1
        for h in range(H):
            g = h // (H // G)
            s = cap_scores(K[:n, g] @ q[t, h], scale, softcap)
            p = np.exp(s - s.max())
            out[t, h] = (p / p.sum()) @ V[:n, g]
    return out


def mix_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def glu_ff(h, W, p):
    g, u = h @ W[p + "mlp.gate"].T, h @ W[p + "mlp.up"].T
    return ((g / (1.0 + np.exp(-g))) * u) @ W[p + "mlp.down"].T


def project_qkv(h, W, p, m, layer_type, positions, eps, v_first):
    """q, k, v of one layer for rows h; returns (q, k, v, v_first)"""
    T = h.shape[0]
    q = (h @ W[p + "mix.q"].T).reshape(T, m["heads"], m["dim"])
    k = (h @ W[p + "mix.k"].T).reshape(T, m["kv_heads"], m["dim"])
    v = (h @ W[p + "mix.v"].T).reshape(T, m["kv_heads"], m["vdim"])
    if layer_type == "attention":
        q, k = rms(q, eps), rms(k, eps)
    else:
        q, k = rotary(q, positions, m["rot"]), rotary(k, positions, m["rot"])
    if m.get("v_mix"):
        if v_first is None:
            v_first = v
        else:
            v = mix_values(v, v_first, float(W[p + "mix.vmix"]))
    return q, k, v, v_first


def forward(cfg, W, tokens):
    """whole sequence at once -> (logits [T][vocab], residual stream after every layer [L][T][width])"""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = np.arange(T)
    x = embed(tokens, None, W, cfg)
    v_first, outs = None, []
    for li, L in enumerate(cfg["layers"]):
        p, m = "l%d." % li, L["mixer"]
        h = rms(x, eps) * W[p + "norm1"]
        q, k, v, v_first = project_qkv(h, W, p, m, L["type"], pos, eps, v_first)
        o = attend(q, k, v, pos, m["scale"], m.get("softcap"))
        if L["type"] == "attention_2":
            o = o * (1.0 / (1.0 + np.exp(-(h @ W[p + "mix.g"].T))))[:, :, None]
        y = (o.reshape(T, -1) @ W[p + "mix.o"].T) * W[p + "ls1"]
        if L.get("mlp"):
            y = y + glu_ff(h, W, p) * W[p + "ls2"]
        x = x + y
        outs.append(x.copy())
    logits = (rms(x, eps) * W["final.norm"]) @ W["head"].T * cfg.get("logit_scale", 1.0)
    return logits, np.array(outs)


class IncrementalOracle:
    """the same model one portion at a time over explicit per-layer K/V lists and a remembered previous token"""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, W
        self.K = [np.zeros((0, L["mixer"]["kv_heads"], L["mixer"]["dim"])) for L in cfg["layers"]]
        self.V = [np.zeros((0, L["mixer"]["kv_heads"], L["mixer"]["vdim"])) for L in cfg["layers"]]
        self.prev, self.n = None, 0

    def step(self, tokens):
        cfg, W, eps = self.cfg, self.W, self.cfg["norm"]["eps"]
        T = len(tokens)
        pos = self.n + np.arange(T)
        x = embed(tokens, self.prev, W, cfg)
        v_first = None
        for li, L in enumerate(cfg["layers"]):
            p, m = "l%d." % li, L["mixer"]
            h = rms(x, eps) * W[p + "norm1"]
            q, k, v, v_first = project_qkv(h, W, p, m, L["type"], pos, eps, v_first)
            self.K[li] = np.concatenate([self.K[li], k])
            self.V[li] = np.concatenate([self.V[li], v])
            o = attend(q, self.K[li], self.V[li], pos, m["scale"], m.get("softcap"))
            if L["type"] == "attention_2":
                o = o * (1.0 / (1.0 + np.exp(-(h @ W[p + "mix.g"].T))))[:, :, None]
            y = (o.reshape(T, -1) @ W[p + "mix.o"].T) * W[p + "ls1"]
            if L.get("mlp"):
                y = y + glu_ff(h, W, p) * W[p + "ls2"]
            x = x + y
        self.prev, self.n = tokens[-1], self.n + T
        return (rms(x, eps) * W["final.norm"]) @ W["head"].T * cfg.get("logit_scale", 1.0)


# ---- small random models ---------------------------------------------------------------------------------------------------
def attention_layer(kind="attention", heads=4, kv_heads=2, dim=16, vdim=16, scale=0.5, softcap=8.0, v_mix=True, ff=48,
                    rot_dims=8, rot_base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "v_mix": v_mix}
    if kind == "attention_2":
        m["rot"] = {"base": rot_base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, width=32, vocab=61, bigram=(13, 7, 5), eps=1e-5, logit_scale=1.5):
    cfg = {"architecture": "Genetar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "layers": layers}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


def tensor_shapes(cfg):
    w, shapes = cfg["width"], {}
    shapes["embed"] = (cfg["vocab"], w)
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        shapes["bigram"] = (bg["buckets"] + 1, w)
    for li, L in enumerate(cfg["layers"]):
        p, m = "l%d." % li, L["mixer"]
        shapes[p + "norm1"] = (w,)
        shapes[p + "mix.q"] = (m["heads"] * m["dim"], w)
        shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], w)
        shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], w)
        shapes[p + "mix.vmix"] = ()
        if L["type"] == "attention_2":
            shapes[p + "mix.g"] = (m["heads"], w)
        shapes[p + "mix.o"] = (w, m["heads"] * m["vdim"])
        shapes[p + "ls1"] = (w,)
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            shapes[p + "mlp.gate"], shapes[p + "mlp.up"], shapes[p + "mlp.down"] = (ff, w), (ff, w), (w, ff)
            shapes[p + "ls2"] = (w,)
    shapes["final.norm"] = (w,)
    shapes["head"] = (cfg["vocab"], w)
    return shapes


def random_weights(cfg, seed=0, qk_gain=1.0):
    """bf16-representable random weights (float64 arrays); qk_gain sharpens the attention of rotary layers"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(("norm1", "final.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith(("ls1", "ls2")):
            a = 0.5 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("vmix"):
            a = np.array(0.15 + 0.5 * rng.random())
        elif name in ("embed", "bigram"):
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / math.sqrt(shape[-1])
            if name.endswith(("mix.q", "mix.k")):
                a = a * qk_gain
        W[name] = bf16_round(a).reshape(shape)
    return W


def write_model(folder, cfg, W):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    header, blobs, off = {}, [], 0
    for name, a in W.items():
        b = to_bf16_bits(np.asarray(a, np.float32)).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(a)), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return folder


def rel_rms(got, want):
    """root mean square of the difference over the root mean square of the expected values"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(np.mean((got - want) ** 2)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))
