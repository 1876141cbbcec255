"""A plain, slow implementation of the dense Llama decoder, for comparison only.

Whole sequences, no cache, no batching, one function per part, numpy on the
CPU.  It shares no code with the engine: it has its own reader for
config.json and safetensors and its own arithmetic.  Every function follows a
formula of the reference (Joakimpalm-Zen/xyntetik-runner, paths within that
project) and cites it.  Values are kept in float32 as the reference keeps
them; sums over many terms (matrix products, norms, softmax) are accumulated
in float64 and rounded once, so that this side of a comparison carries less
rounding error than either engine path.

Where the reference's own CPU build anchors these formulas, see
tests/golden/README.md; positions, frequency tables and angles are computed in
float32 exactly as src/model.c does, because an engine that computes them the
same way must agree to the last bits of the angle.

Layout notes.  The reference's llama GGUFs carry Q/K rows permuted for
adjacent-pair rotation (src/model.c:1464-1466); a config.json + safetensors
folder carries them unpermuted, for which the same function rotates the pairs
(j, j + half) -- the reference's `rope_neox` branch (src/model.c:3523-3525).
Scores are the same either way.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------
# reading a model folder (own reader; the engine's is not used)
# --------------------------------------------------------------------------
def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    # bf16 is the top 16 bits of a float32 (src/fp16.h:52-66)
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_folder(model_dir: str):
    """Returns (config dict, {name: float32 array})."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    path = os.path.join(model_dir, "model.safetensors")
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        blob = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        b, e = ent["data_offsets"]
        raw = blob[b:e]
        if ent["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(F32)
        elif ent["dtype"] == "BF16":
            a = _bf16_to_f32(np.frombuffer(raw, dtype="<u2"))
        elif ent["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(F32)
        else:
            raise ValueError(f"{name}: dtype {ent['dtype']}")
        out[name] = a.reshape(ent["shape"])
    return cfg, out


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def matvec_rows(x: np.ndarray, w: np.ndarray, bias=None) -> np.ndarray:
    """y[t][r] = sum_i W[r][i] * x[t][i] (+ b[r]): src/model.c:3426-3506 (`matvec_b`),
    float32 values, one rounding of a wide sum."""
    y = x.astype(np.float64) @ np.asarray(w, dtype=np.float64).T           # (no copy when w is wide already)
    if bias is not None:
        y = y + bias.astype(np.float64)
    return y.astype(F32)


def embed(ids, table: np.ndarray) -> np.ndarray:
    """x[b] = E[id_b]; an id outside [0, V) is replaced by 0; no scale for llama
    (src/model.c:6148-6162, embd_scale = 1 at src/model.c:1467)."""
    ids = np.asarray(ids, dtype=np.int64)
    ids = np.where((ids < 0) | (ids >= table.shape[0]), 0, ids)
    return table[ids].astype(F32)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """o = x * 1/sqrt(sum(x^2)/n + eps) * w, per row (src/model.c:3386-3392)."""
    xx = x.astype(np.float64)
    ss = (xx * xx).sum(axis=-1, keepdims=True)
    r = 1.0 / np.sqrt(ss / x.shape[-1] + np.float64(F32(eps)))
    return (xx * r * w.astype(np.float64)).astype(F32)


def rope_inv_freq(theta: float, rope_dim: int, scaling=None) -> np.ndarray:
    """inv_freq[j] = theta^(-2j/rope_dim) in float32 (`powf`, src/model.c:288-289), then divided by
    per-frequency factors where the model has them (src/model.c:291-297).

    The reference reads those factors from a tensor that the converter wrote.  For
    rope_scaling of type llama3 they are, by wavelength lam_j = 2*pi/f_j:
      lam_j < orig/high_freq_factor  -> 1
      lam_j > orig/low_freq_factor   -> factor
      else, s = (orig/lam_j - low)/(high - low):  f_j' = (1-s) f_j/factor + s f_j,
    i.e. divisor f_j / f_j'.
    """
    half = rope_dim // 2
    j = np.arange(half, dtype=F32)
    expo = (F32(-2.0) * j / F32(rope_dim)).astype(F32)
    inv = np.power(F32(theta), expo).astype(F32)
    if scaling is None:
        return inv
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind == "linear":                       # every frequency divided by the factor, in float32 (src/model.c:361-362)
        return (inv / F32(scaling["factor"])).astype(F32)
    if kind != "llama3":
        raise ValueError(f"rope_scaling {kind}")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(inv)
    for i in range(half):
        f = float(inv[i])
        lam = 2.0 * math.pi / f
        if lam < orig / high:
            div = 1.0
        elif lam > orig / low:
            div = factor
        else:
            s = (orig / lam - low) / (high - low)
            div = f / ((1.0 - s) * f / factor + s * f)
        out[i] = F32(inv[i] / F32(div))       # the reference divides in float32 (src/model.c:295)
    return out


def rope_apply(v: np.ndarray, positions: np.ndarray, inv_freq: np.ndarray, adjacent: bool = False, mscale: float = 1.0) -> np.ndarray:
    """v: [T, heads, hd].  a = pos * f_j in float32; (c, s) = (cos a, sin a) * mscale; (x0, x1) -> (x0 c - x1 s,
    x0 s + x1 c) on the pairs (j, j + half), the reference's `rope_neox` branch, or on (2j, 2j + 1) with
    `adjacent`, its branch for files with permuted rows (src/model.c:3514-3532; mscale src/model.c:283, 375)."""
    T, nh, hd = v.shape
    half = inv_freq.shape[0]
    a = (positions.astype(F32)[:, None] * inv_freq[None, :]).astype(F32)      # float32 product
    c = (np.cos(a.astype(np.float64)).astype(F32) * F32(mscale)).astype(F32)[:, None, :]
    s = (np.sin(a.astype(np.float64)).astype(F32) * F32(mscale)).astype(F32)[:, None, :]
    out = v.copy()
    i0 = np.arange(0, 2 * half, 2) if adjacent else np.arange(half)
    i1 = i0 + 1 if adjacent else i0 + half
    x0, x1 = v[:, :, i0], v[:, :, i1]
    out[:, :, i0] = (x0 * c - x1 * s).astype(F32)
    out[:, :, i1] = (x0 * s + x1 * c).astype(F32)
    return out


def softmax_rows(s: np.ndarray) -> np.ndarray:
    """m = max; e = exp(s - m); a = e / sum(e) (src/model.c:3409-3415)."""
    s = s.astype(np.float64)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / e.sum(axis=-1, keepdims=True)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window=None) -> np.ndarray:
    """q: [T, H, hd], k, v: [T, K, hd] of one sequence from position 0.  For the query at position p
    and head h, with kvh = h / (H/K): s_t = (q . k_t) * scale for t0 <= t <= p, softmax, then
    o = sum_t a_t v_t (src/model.c:3548-3589; causal by loop bound, t0 = 0 without a window,
    src/model.c:6326; with a window of w keys t0 = max(0, p - w + 1))."""
    T, H, hd = q.shape
    K = k.shape[1]
    mul = H // K
    out = np.zeros((T, H, hd), dtype=F32)
    for h in range(H):
        kvh = h // mul
        kk = k[:, kvh, :].astype(np.float64)
        vv = v[:, kvh, :].astype(np.float64)
        for p in range(T):
            t0 = 0 if window is None else max(0, p - window + 1)
            s = (kk[t0:p + 1] @ q[p, h].astype(np.float64)) * np.float64(F32(scale))
            a = softmax_rows(s[None, :])[0]
            out[p, h] = (a @ vv[t0:p + 1]).astype(F32)
    return out


def attention_in_blocks(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window=None, block: int = 256) -> np.ndarray:
    """The same function as ``attention`` for long sequences: per head, a block of queries at a time against all
    keys up to the block's last position, the keys a query may not see masked out before the softmax
    (the reference's loop bounds t0..p, src/model.c:3556-3573, as a mask)."""
    T, H, hd = q.shape
    K = k.shape[1]
    mul = H // K
    out = np.zeros((T, H, hd), dtype=F32)
    sc = np.float64(F32(scale))
    for h in range(H):
        kk = k[:, h // mul, :].astype(np.float64)
        vv = v[:, h // mul, :].astype(np.float64)
        for p0 in range(0, T, block):
            p1 = min(T, p0 + block)
            t_lo = 0 if window is None else max(0, p0 - window + 1)
            s = (q[p0:p1, h].astype(np.float64) @ kk[t_lo:p1].T) * sc
            pos = np.arange(p0, p1)[:, None]
            key = np.arange(t_lo, p1)[None, :]
            hidden = key > pos
            if window is not None:
                hidden |= key < pos - window + 1
            s = np.where(hidden, -np.inf, s)
            out[p0:p1, h] = (softmax_rows(s) @ vv[t_lo:p1]).astype(F32)
    return out


def swiglu(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """h = g / (1 + exp(-g)) * u, and 0 where g < -80 (src/model.c:4451-4452)."""
    gg = g.astype(np.float64)
    with np.errstate(over="ignore"):
        h = gg / (1.0 + np.exp(-gg)) * u.astype(np.float64)
    h = np.where(gg < -80.0, 0.0, h)
    return h.astype(F32)


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
class PlainLlama:
    def __init__(self, model_dir: str = None, *, config: dict = None, tensors: dict = None):
        """From a folder, or from config.json's keys as a dict plus {tensor name: float32 array}."""
        if model_dir is not None:
            self.cfg, self.w = read_folder(model_dir)
        else:
            self.cfg, self.w = dict(config), dict(tensors)
        self._wide = {}         # float64 copies of the matrices, made once (big models would convert them at every call)
        c = self.cfg
        self.d = c["hidden_size"]
        self.L = c["num_hidden_layers"]
        self.H = c["num_attention_heads"]
        self.K = c.get("num_key_value_heads") or self.H
        self.hd = c.get("head_dim") or self.d // self.H
        self.eps = c["rms_norm_eps"]
        self.inv_freq = rope_inv_freq(c.get("rope_theta", 10000.0), self.hd, c.get("rope_scaling"))
        self.scale = 1.0 / math.sqrt(self.hd)          # src/model.h:464-467
        self.window = c.get("sliding_window")
        self.layer_types = c.get("layer_types")

    def _window(self, layer):
        if self.window is None:
            return None
        if self.layer_types is None or self.layer_types[layer] == "sliding_attention":
            return self.window
        return None

    def mat(self, name: str) -> np.ndarray:
        if name not in self._wide:
            self._wide[name] = self.w[name].astype(np.float64)
        return self._wide[name]

    def layer(self, x: np.ndarray, l: int, positions: np.ndarray) -> np.ndarray:
        """x -> norm -> attention -> +x -> norm -> feed-forward -> +x (src/model.c:6206-6423)."""
        w, p = self.w, f"model.layers.{l}."
        T = x.shape[0]
        attend = attention if T <= 256 else attention_in_blocks
        bias = (lambda n: w.get(p + n)) if self.cfg.get("attention_bias") else (lambda n: None)
        xb = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)
        q = matvec_rows(xb, self.mat(p + "self_attn.q_proj.weight"), bias("self_attn.q_proj.bias")).reshape(T, self.H, self.hd)
        k = matvec_rows(xb, self.mat(p + "self_attn.k_proj.weight"), bias("self_attn.k_proj.bias")).reshape(T, self.K, self.hd)
        v = matvec_rows(xb, self.mat(p + "self_attn.v_proj.weight"), bias("self_attn.v_proj.bias")).reshape(T, self.K, self.hd)
        q = rope_apply(q, positions, self.inv_freq)          # after projection, before the cache (src/model.c:6276-6299)
        k = rope_apply(k, positions, self.inv_freq)
        o = attend(q, k, v, self.scale, self._window(l)).reshape(T, self.H * self.hd)
        x = (x + matvec_rows(o, self.mat(p + "self_attn.o_proj.weight"), bias("self_attn.o_proj.bias"))).astype(F32)
        xb = rmsnorm(x, w[p + "post_attention_layernorm.weight"], self.eps)
        h = swiglu(matvec_rows(xb, self.mat(p + "mlp.gate_proj.weight")), matvec_rows(xb, self.mat(p + "mlp.up_proj.weight")))
        x = (x + matvec_rows(h, self.mat(p + "mlp.down_proj.weight"))).astype(F32)
        return x

    def hidden(self, ids) -> np.ndarray:
        x = embed(ids, self.w["model.embed_tokens.weight"])
        pos = np.arange(len(ids), dtype=np.int64)
        for l in range(self.L):
            x = self.layer(x, l, pos)
        return x

    def logits(self, ids, rows=None) -> np.ndarray:
        """Logits at every position of the whole sequence (or at the positions `rows`): final norm, then the
        head, which is the embedding table when the model has no lm_head tensor (src/model.c:2353-2354, 6478-6481)."""
        x = self.hidden(ids)
        if rows is not None:
            x = x[np.asarray(rows, dtype=np.int64)]
        xb = rmsnorm(x, self.w["model.norm.weight"], self.eps)
        head = self.mat("lm_head.weight" if "lm_head.weight" in self.w else "model.embed_tokens.weight")
        return matvec_rows(xb, head)

    def generate_greedy(self, ids, n_new: int):
        """Argmax decoding, first index on ties (src/sample.c:169-172), recomputing everything each step."""
        ids = list(ids)
        out = []
        for _ in range(n_new):
            lg = self.logits(ids)[-1]
            t = int(np.argmax(lg))
            out.append(t)
            ids.append(t)
        return out


# --------------------------------------------------------------------------
# sampling (src/sample.c), on given logits
# --------------------------------------------------------------------------
def score_logprobs(logits: np.ndarray, tokens) -> np.ndarray:
    """Teacher-forced scoring (src/main.c:1395-1405): for position i, lp = lg[tokens[i + 1]] - (max + log(sum exp(lg - max))),
    maximum and result in float32, the sum in double.  logits: [T, vocab] of the whole sequence; returns T - 1 values."""
    out = np.zeros(len(tokens) - 1, dtype=F32)
    for i in range(len(tokens) - 1):
        lg = logits[i].astype(F32)
        mx = lg.max()
        total = np.exp((lg - mx).astype(F32)).astype(np.float64).sum()
        out[i] = F32(lg[tokens[i + 1]] - F32(mx + F32(np.log(F32(total)))))
    return out


def xorshift64(state: int):
    """src/sample.c:13-17."""
    m = (1 << 64) - 1
    x = state & m
    x ^= (x << 13) & m
    x ^= x >> 7
    x ^= (x << 17) & m
    return x


def uniform_from_state(state: int) -> float:
    """(x >> 40) / 2^24 (src/sample.c:18-20)."""
    return float(F32((state >> 40) / 16777216.0))


def sample_chain(logits: np.ndarray, r: float, temp: float, top_k: int = 0, top_p: float = 1.0,
                 min_p: float = 0.0, repeat_penalty: float = 1.0, recent=(), with_margin: bool = False,
                 distance_of=None):
    """The reference's chain on one row (src/sample.c:141-329, `pick_scaled` :86-127):
    penalty on recent tokens (only when temp > 0), greedy for temp <= 0, scale by 1/temp, keep the
    top_k by (logit descending, id ascending), softmax over the survivors, top-p prefix, min-p floor,
    then the first candidate whose cumulative probability exceeds r."""
    lg = logits.astype(F32).copy()
    V = lg.shape[0]
    if temp > 0 and repeat_penalty != 1.0:
        for t in recent:
            if 0 <= t < V:
                lg[t] = lg[t] / F32(repeat_penalty) if lg[t] > 0 else lg[t] * F32(repeat_penalty)
    if temp <= 0:
        if distance_of is not None:
            return float(lg.max() - lg[distance_of])       # how far below the best logit the given token lies
        if with_margin:
            top2 = np.sort(lg)[-2:]
            return int(np.argmax(lg)), float(top2[1] - top2[0])
        return int(np.argmax(lg))
    sc = (lg / F32(temp)).astype(F32)
    order = np.lexsort((np.arange(V), -sc.astype(np.float64)))
    k = top_k if 0 < top_k < V else V
    order = order[:k]
    p = np.exp((sc[order] - sc[order[0]]).astype(np.float64))
    p = p / p.sum()
    if top_p < 1.0:
        cum = np.cumsum(p)
        cut = int(np.searchsorted(cum, top_p, side="left")) + 1
        cut = min(cut, k)
        order, p = order[:cut], p[:cut] / p[:cut].sum()
    if min_p > 0.0:
        keep = 1
        while keep < len(p) and p[keep] >= min_p * p[0]:
            keep += 1
        order, p = order[:keep], p[:keep] / p[:keep].sum()
    cum = np.cumsum(p)
    idx = int(np.searchsorted(cum, r, side="right"))
    idx = min(idx, len(order) - 1)
    if distance_of is not None:
        # how far the draw lies outside the given token's interval of the cumulative distribution
        where = np.nonzero(order == distance_of)[0]
        if len(where) == 0:
            return float("inf")
        j = int(where[0])
        lo, hi = (cum[j - 1] if j > 0 else 0.0), cum[j]
        return float(max(lo - r, r - hi, 0.0))
    if with_margin:
        # distance of the draw to the nearest edge of the picked candidate's interval: a pick is only
        # comparable between two implementations when the draw is not on an edge
        lo = cum[idx - 1] if idx > 0 else 0.0
        return int(order[idx]), float(min(r - lo, cum[idx] - r))
    return int(order[idx])
