"""Plain, slow Llama decoder used as the oracle of every numerics test.

It rests on the formulas of the reference's CPU path (go-pherence, Go): that
project cannot be compiled or imported here (no Go toolchain, three external
modules, no network), so nothing below was compared against its binaries.  What
it takes from the reference are the formulas, cited per function as
``file:line`` within that project, and a handful of small vectors from its own
unit tests (see tests/test_plain.py).  llama3 frequency scaling, batching,
sampling with a temperature and stop tokens have no counterpart there.

Whole sequences, no cache, one function for each part, NumPy only.  It shares
no code with the package: it has its own config reading, its own safetensors
reader and its own random-number function.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# configuration (model/llama.go:36-49 for the keys, :223-237 for the defaults)
# --------------------------------------------------------------------------
def read_config(folder):
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    return normalise_config(raw)


def normalise_config(raw):
    cfg = dict(raw)
    if not cfg.get("rms_norm_eps"):
        cfg["rms_norm_eps"] = 1e-5                      # model/llama.go:223-225
    if not cfg.get("head_dim"):
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]  # :235-237
    if not cfg.get("num_key_value_heads"):
        cfg["num_key_value_heads"] = cfg["num_attention_heads"]
    if not cfg.get("rope_theta"):
        cfg["rope_theta"] = 10000.0
    cfg.setdefault("tie_word_embeddings", False)
    cfg.setdefault("rope_scaling", None)
    return cfg


# --------------------------------------------------------------------------
# weights: a minimal safetensors reader (loader/safetensors/safetensors.go:78-143
# for the container: u64 little-endian header length, JSON header, raw bytes)
# --------------------------------------------------------------------------
def _bf16_to_f32(u16):
    return (u16.astype(np.uint32) << 16).view(np.float32)   # safetensors.go:258-268


def read_safetensors(path):
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = blob[base + a: base + b]
        dt = meta["dtype"]
        if dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(F32)
        elif dt == "BF16":
            arr = _bf16_to_f32(np.frombuffer(raw, dtype="<u2"))
        elif dt == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(F32)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(meta["shape"])
    return out


def read_model(folder):
    """(config, tensors by HF name as float32)."""
    return read_config(folder), read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(table, tokens):
    """x = E[tok,:], no scaling for llama (model/inference_helpers.go:9-34)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    if tokens.min() < 0 or tokens.max() >= table.shape[0]:
        raise IndexError("token id outside the vocabulary")
    return table[tokens].astype(F32)


def rms_norm(x, w, eps):
    """y_i = w_i * x_i * (1/sqrt(mean(x^2)+eps)); the sum of squares is a
    float32 running sum, the square root is taken in float64 and rounded
    (backends/simd/vec.go:72-85,117-119)."""
    x = np.asarray(x, dtype=F32)
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        row = x[r]
        ss = np.cumsum(row * row, dtype=F32)[-1]      # the float32 running sum, left to right
        s = F32(1.0) / F32(math.sqrt(float(F32(ss / F32(row.shape[0])) + F32(eps))))
        out[r] = (w.astype(F32) * row) * s
    return out


def rope_inv_freq(cfg):
    """f_i = theta^(-2i/hd) in float64 (model/llama.go:856-858).  The llama3
    rescaling of the frequencies has no counterpart in the reference; it is the
    published rule: keep short wavelengths, divide long ones by `factor`, blend
    linearly in between."""
    hd = cfg["head_dim"]
    theta = float(cfg["rope_theta"])
    f = np.array([1.0 / math.pow(theta, (2 * i) / hd) for i in range(hd // 2)], dtype=np.float64)
    rs = cfg.get("rope_scaling")
    if rs:
        kind = rs.get("rope_type", rs.get("type"))
        if kind != "llama3":
            raise ValueError(f"plain implementation: rope_scaling type {kind}")
        factor = float(rs["factor"])
        low = float(rs["low_freq_factor"])
        high = float(rs["high_freq_factor"])
        p0 = float(rs["original_max_position_embeddings"])
        out = f.copy()
        for i, fi in enumerate(f):
            wavelen = 2.0 * math.pi / fi
            if wavelen < p0 / high:
                out[i] = fi
            elif wavelen > p0 / low:
                out[i] = fi / factor
            else:
                smooth = (p0 / wavelen - low) / (high - low)
                out[i] = (1.0 - smooth) * fi / factor + smooth * fi
        f = out
    return f


def rope(x, positions, inv_freq, n_heads, hd):
    """Half-split pairs (i, i+hd/2); the angle pos*f_i is float64, cos and sin
    are rounded to float32 (model/llama.go:838-865 table, :1556-1589 apply)."""
    x = np.asarray(x, dtype=F32).reshape(len(positions), n_heads, hd).copy()
    half = hd // 2
    for t, pos in enumerate(positions):
        ang = float(pos) * inv_freq
        c = np.cos(ang).astype(F32)
        s = np.sin(ang).astype(F32)
        a = x[t, :, :half].copy()
        b = x[t, :, half:].copy()
        x[t, :, :half] = a * c - b * s
        x[t, :, half:] = a * s + b * c
    return x.reshape(len(positions), n_heads * hd)


def linear(x, w):
    """y = x . W^T with W stored [out, in] (gemvNT, model/llama.go:1516-1536)."""
    return (np.asarray(x, dtype=F32) @ np.asarray(w, dtype=F32).T).astype(F32)


def causal_gqa_attention(q, k, v, n_heads, n_kv, hd, window=None, scale=None):
    """Scores (q.k)*scale with scale = float32(1/sqrt(hd)) applied after the dot,
    softmax as exp(float64(s-max)) rounded to float32 and normalised by 1/sum,
    then the weighted sum of V; head h reads KV head h // (n_heads/n_kv)
    (model/llama.go:1603-1661).  Token t sees keys 0..t (and, with `window`,
    only the last `window` of them; the reference has no window for llama).
    `scale` replaces 1/sqrt(hd) (the reference's function takes it as an argument:
    gqaAttentionScale, model/attention_test.go:57)."""
    T = q.shape[0]
    q = q.reshape(T, n_heads, hd)
    k = k.reshape(T, n_kv, hd)
    v = v.reshape(T, n_kv, hd)
    group = n_heads // n_kv
    scale = F32(1.0 / math.sqrt(hd)) if scale is None else F32(scale)
    out = np.zeros((T, n_heads, hd), dtype=F32)
    for h in range(n_heads):
        kvh = h // group
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, kvh, :] @ q[t, h, :]).astype(F32) * scale
            m = s.max()
            e = np.exp((s - m).astype(np.float64)).astype(F32)
            z = F32(0.0)
            for ev in e:
                z = F32(z + ev)
            p = e * (F32(1.0) / z)
            out[t, h, :] = (p[:, None] * v[lo:t + 1, kvh, :]).sum(axis=0, dtype=F32)
    return out.reshape(T, n_heads * hd)


def silu_mul(gate, up):
    """h = gate/(1+exp(-gate)) * up, exp in float64 (backends/simd/vec.go:52-59)."""
    gate = np.asarray(gate, dtype=F32)
    s = gate / (F32(1.0) + np.exp(-gate.astype(np.float64)).astype(F32))
    return (s * np.asarray(up, dtype=F32)).astype(F32)


def swiglu_mlp(x, wg, wu, wd):
    """down(silu(gate(x)) * up(x)) (model/llama.go:1361-1401)."""
    return linear(silu_mul(linear(x, wg), linear(x, wu)), wd)


def _no_trace(op, value):
    pass


def attention_block(x, positions, p, cfg, inv_freq, w, window=None, trace=_no_trace):
    """q,k,v projections, RoPE on q and k, causal GQA attention, output
    projection (model/llama.go:1111-1137, 1230-1233, 1259-1297).  `trace(op,
    value)` receives the values the reference hands to its per-op hook under
    the same names (model/llama.go:1147-1153 q k v, :1236-1241 q_attn k_attn,
    :1285-1287 attn, :1298-1300 o)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = linear(x, w[p + "self_attn.q_proj.weight"])
    k = linear(x, w[p + "self_attn.k_proj.weight"])
    v = linear(x, w[p + "self_attn.v_proj.weight"])
    trace("q", q); trace("k", k); trace("v", v)
    q = rope(q, positions, inv_freq, nh, hd)
    k = rope(k, positions, inv_freq, nkv, hd)
    trace("q_attn", q); trace("k_attn", k)
    a = causal_gqa_attention(q, k, v, nh, nkv, hd, window=window)
    trace("attn", a)
    o = linear(a, w[p + "self_attn.o_proj.weight"])
    trace("o", o)
    return o


def decoder_layer(x, positions, layer, cfg, inv_freq, w, trace=_no_trace):
    """Pre-norm residual block: x += attn(norm1(x)); x += mlp(norm2(x))
    (model/llama.go:1087-1097, 1311-1314, 1425).  `trace(op, value)`: the
    reference's per-op hook names (model/llama.go:1089-1101 hidden_in normed,
    :1351-1353 mlp_input, :1378-1391 gate_pre up gate_act, :1408-1410 down,
    :1426-1428 hidden_post_ffn)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    trace("hidden_in", x)
    n = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    trace("normed", n)
    x = (x + attention_block(n, positions, p, cfg, inv_freq, w, trace=trace)).astype(F32)
    n2 = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    trace("mlp_input", n2)
    gate, up = linear(n2, w[p + "mlp.gate_proj.weight"]), linear(n2, w[p + "mlp.up_proj.weight"])
    trace("gate_pre", gate); trace("up", up)
    act = silu_mul(gate, up)
    trace("gate_act", act)
    d = linear(act, w[p + "mlp.down_proj.weight"])
    trace("down", d)
    x = (x + d).astype(F32)
    trace("hidden_post_ffn", x)
    return x


def lm_head(x, cfg, w):
    """Final RMSNorm then logits_v = sum_k x_k*LM[v,k]; LM is lm_head.weight if
    the file has it, else embed_tokens.weight (model/cpu_decode_step.go:31-44,
    model/inference_helpers.go:145-148, model/llama.go:490-494)."""
    xf = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    table = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(xf, table)


def forward(cfg, w, tokens, layer_order=None, trace=None):
    """Logits [T, V] of one whole sequence (model/llama.go:1047-1473 run for
    every position).  `layer_order` lists the layers to run (default 0..L-1).
    `trace(layer, op, value)` receives every layer's named intermediate values."""
    tokens = list(tokens)
    positions = list(range(len(tokens)))
    inv_freq = rope_inv_freq(cfg)
    x = embed(w["model.embed_tokens.weight"], tokens)
    order = range(cfg["num_hidden_layers"]) if layer_order is None else layer_order
    for layer in order:
        layer_trace = _no_trace if trace is None else (lambda op, value, layer=layer: trace(layer, op, value))
        x = decoder_layer(x, positions, layer, cfg, inv_freq, w, trace=layer_trace)
    return lm_head(x, cfg, w)


# --------------------------------------------------------------------------
# sampling and generation
# --------------------------------------------------------------------------
def argmax_first(logits):
    """Strict '>' scan: the lowest index wins ties (model/inference_helpers.go:153-166)."""
    best, best_v = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > best_v:
            best, best_v = i, logits[i]
    return best


_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform(seed, sequence, step):
    """Counter-based uniform in [0,1) with 24 random bits: a function of
    (seed, sequence index, step) only, so a draw does not depend on what else
    is in the batch.  Ours; the reference samples greedily only."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ ((sequence * 0xD1B54A32D192ED03) & _M64))
    z = _mix64(z ^ ((step * 0x8CB92BA72F3D8DD7) & _M64))
    return (z >> 40) * (1.0 / (1 << 24))


def temperature_probs(logits, temperature):
    """softmax(logits / T) in float32 statistics (max-subtracted)."""
    z = np.asarray(logits, dtype=F32) / F32(temperature)
    z = z - z.max()
    e = np.exp(z.astype(np.float64))
    return e / e.sum()


def sample_temperature(logits, temperature, u):
    """Inverse CDF: the first token whose cumulative probability exceeds u."""
    cdf = np.cumsum(temperature_probs(logits, temperature))
    idx = int(np.searchsorted(cdf, u, side="right"))
    return min(idx, len(cdf) - 1)


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0, sequence=0, stop=()):
    """Token-by-token generation by recomputing the whole sequence each time.
    Returns the new tokens only; a stop token is kept and ends the sequence."""
    seq = list(prompt)
    new = []
    for step in range(max_new_tokens):
        logits = forward(cfg, w, seq)[-1]
        if temperature > 0:
            tok = sample_temperature(logits, temperature, uniform(seed, sequence, step))
        else:
            tok = argmax_first(logits)
        new.append(tok)
        seq.append(tok)
        if tok in stop:
            break
    return new
