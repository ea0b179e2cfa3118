"""Model folders (config.json + model.safetensors) for the architectures the library opens by name: a writer, the
tensor table of the Genetar architecture, and random bf16 weights of a given shape for benchmarks and smoke runs.

safetensors layout: 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets
relative to the end of the header), then the tensor data.
"""
import json
import math
import os
import struct

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def genetar_config(width, ff, n_layers, heads, kv_heads, head_dim, vocab, *, buckets=4099, rot_dims=None, eps=1e-5,
                   softcap=50.0, logit_scale=1.0, pattern=("attention", "attention_2")):
    """layers alternate through `pattern`; every layer mixes values and has a dense SiLU-GLU feed-forward"""
    layers = []
    for i in range(n_layers):
        kind = pattern[i % len(pattern)]
        m = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": 1.0 / math.sqrt(head_dim),
             "softcap": softcap, "v_mix": True}
        if kind == "attention_2":
            m["rot"] = {"base": 500000.0, "dims": rot_dims or head_dim // 2,
                        "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
        layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Genetar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 8191, "mul_cur": 127}}, "layers": layers}


def genetar_tensors(cfg):
    """[(name, shape, kind)]; kind: 'matrix' (fan-in scaled), 'table', 'ones', 'scalar'"""
    w, out = cfg["width"], [("embed", (cfg["vocab"], cfg["width"]), "table")]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out.append(("bigram", (bg["buckets"] + 1, w), "table"))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out += [(p + "norm1", (w,), "ones"), (p + "mix.q", (m["heads"] * m["dim"], w), "matrix"),
                (p + "mix.k", (m["kv_heads"] * m["dim"], w), "matrix"), (p + "mix.v", (m["kv_heads"] * m["vdim"], w), "matrix"),
                (p + "mix.vmix", (), "scalar")]
        if L["type"] == "attention_2":
            out.append((p + "mix.g", (m["heads"], w), "matrix"))
        out += [(p + "mix.o", (w, m["heads"] * m["vdim"]), "matrix"), (p + "ls1", (w,), "ones")]
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            out += [(p + "mlp.gate", (ff, w), "matrix"), (p + "mlp.up", (ff, w), "matrix"), (p + "mlp.down", (w, ff), "matrix"),
                    (p + "ls2", (w,), "ones")]
    out += [("final.norm", (w,), "ones"), ("head", (cfg["vocab"], w), "matrix")]
    return out


def genetar_param_bytes(cfg, bytes_per_weight=2):
    """bytes a decode step streams: every matrix once, one row of each table"""
    total = 0
    for name, shape, kind in genetar_tensors(cfg):
        n = int(np.prod(shape)) if shape else 1
        total += (shape[1] if kind == "table" else n) * bytes_per_weight
    return total


def genetar_matmul_flops_per_token(cfg):
    return sum(2 * int(np.prod(shape)) for name, shape, kind in genetar_tensors(cfg) if kind == "matrix")


def write_random_genetar(folder, cfg, seed=0):
    """random bf16 weights, streamed to disk tensor by tensor (a full-size model does not have to fit in host memory twice)"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    table, header, off = genetar_tensors(cfg), {}, 0
    for name, shape, _ in table:
        n = (int(np.prod(shape)) if shape else 1) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    rng = np.random.default_rng(seed)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for name, shape, kind in table:
            n = int(np.prod(shape)) if shape else 1
            if kind == "ones":
                a = 1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif kind == "scalar":
                a = np.array([0.25], np.float32)
            else:
                a = rng.standard_normal(n, dtype=np.float32)
                if kind == "matrix":
                    a *= np.float32(1.0 / math.sqrt(shape[-1]))
            f.write(f32_to_bf16_bits(a).tobytes())
    return folder
