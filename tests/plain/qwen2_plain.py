"""A plain, slow implementation of the Qwen2 dense decoder, used only as the oracle of the tests.

Whole sequences, no cache, no batching, one function for each part, float64 on the CPU.
It shares no code with the package under test: it has its own safetensors reader, its own
config reading and its own arithmetic.  Every function cites the file and lines of
tzar-beep/Tensorline that fix its formula (paths are relative to that project's root).  Where
that project delegates a formula to an installed package (the SwiGLU feed-forward, the rotary
frequency table), the standard definition is written out here and said so.

The sliding-window option of the architecture's config.json (`use_sliding_window`,
`sliding_window`, `max_window_layers`) is not run by tzar-beep/Tensorline (its attention is
always full, tensorline/paged.py:230-237).  It is defined here by formula: in a window layer a
query at position p sees the keys at positions j with 0 <= p - j < sliding_window; layers with
index >= max_window_layers are window layers.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """The safetensors container: u64 header length, JSON header, raw little-endian data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        buf = bytearray(raw[8 + n + a:8 + n + b])
        t = torch.frombuffer(buf, dtype=_ST_DTYPES[meta["dtype"]]) if buf else torch.empty(0, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


class PlainQwen2:
    """Weights and constants of one model folder, all weights widened to float64."""

    def __init__(self, folder):
        folder = Path(folder)
        c = json.loads((folder / "config.json").read_text())
        self.cfg = c
        self.L = c["num_hidden_layers"]
        self.H = c["hidden_size"]
        self.nq = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nq)
        self.d = c.get("head_dim") or self.H // self.nq          # tensorline/manager.py:50
        self.eps = c.get("rms_norm_eps", 1e-6)
        theta = c.get("rope_theta")
        if theta is None and isinstance(c.get("rope_parameters"), dict):
            theta = c["rope_parameters"].get("rope_theta")
        self.theta = 10000.0 if theta is None else float(theta)
        self.tied = bool(c.get("tie_word_embeddings", False))
        self.window = [None] * self.L
        if c.get("use_sliding_window", False) and c.get("sliding_window"):
            for i in range(self.L):
                if i >= c.get("max_window_layers", self.L):
                    self.window[i] = int(c["sliding_window"])
        self.w = {k: v.to(F64) for k, v in read_safetensors(folder / "model.safetensors").items()}

    @classmethod
    def from_tensors(cls, config: dict, tensors: dict, dtype=F64):
        """The same from an in-memory config.json dictionary and name -> tensor map (no files)."""
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            (Path(tmp) / "config.json").write_text(json.dumps(config))
            (Path(tmp) / "model.safetensors").write_bytes(struct.pack("<Q", 2) + b"{}")
            m = cls(tmp)
        m.w = {k: v.detach().cpu().to(dtype) for k, v in tensors.items()}
        return m

    def layer(self, i, name):
        return self.w[f"model.layers.{i}.{name}"]


# ---------------------------------------------------------------- parts, one function each

def embedding(table, ids):
    """x[t] = E[ids[t]]; no scaling, nothing added (tensorline/paged.py:240)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """out = x * rsqrt(mean(x^2) + eps) * w; the weight multiplies, no 1+w
    (tensorline/fused.py:29-32)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def linear(x, weight, bias=None):
    """y = x W^T (+ b); weights are [out, in] (tensorline/quant.py:3, tensorline/paged.py:248-250)."""
    y = x @ weight.T
    return y if bias is None else y + bias


def rope_cos_sin(positions, d, theta):
    """cos/sin of angle[p, i] = p * theta^(-2i/d), i in [0, d/2).  The frequency table is
    delegated by tzar-beep/Tensorline to an installed package (tensorline/paged.py:241-242); the
    standard table is used.  As there, the inverse frequencies and the angle are 32-bit values
    (the product p * inv_freq is rounded to float32); their cosine and sine are then taken
    exactly.  Both halves of a row use the same d/2 values (tests/test_quant.py:116-118)."""
    i = torch.arange(0, d, 2, dtype=F64)
    inv_freq = (float(theta) ** (-i / d)).to(torch.float32)
    p = torch.as_tensor(positions, dtype=torch.float32)
    angle = (p[:, None] * inv_freq[None, :]).to(F64)           # the float32 product, widened
    return torch.cos(angle), torch.sin(angle)


def apply_rope(x, cos, sin):
    """Rotate-half: a = x[..., :d/2], b = x[..., d/2:];  out = (a cos - b sin, b cos + a sin)
    (tensorline/fused.py:47-51, equivalently x*cos + rotate_half(x)*sin, fused.py:83-85).
    x is [T, heads, d]; cos, sin are [T, d/2]."""
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((a * c - b * s, b * c + a * s), dim=-1)


def attention(q, k, v, window=None):
    """Causal grouped-query attention over one whole sequence.
    q [T, nq, d], k and v [T, nkv, d].  Query head j uses KV head j // (nq/nkv)
    (tensorline/paged_attn.py:34, tensorline/paged.py:156).  scale = d^-1/2
    (tensorline/paged.py:119), key j visible to query p iff j <= p (tensorline/paged.py:237),
    masked scores are -inf (tensorline/paged_attn.py:48), softmax over keys, o = P V.
    `window`: see the module docstring."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    scale = d ** -0.5
    out = torch.empty_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible = visible & (pos[:, None] - pos[None, :] < window)
    for j in range(nq):
        kk, vv = k[:, j // g], v[:, j // g]
        s = (q[:, j] @ kk.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, j] = p @ vv
    return out


def swiglu(h, w_gate, w_up, w_down):
    """y = (silu(h Wg^T) * (h Wu^T)) Wd^T with silu(z) = z / (1 + e^-z).  tzar-beep/Tensorline
    calls the installed package's module here (tensorline/paged.py:276); shapes are those of
    tensorline/manager.py:53-54; this is the standard SwiGLU, no biases."""
    g = h @ w_gate.T
    u = h @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


def decoder_layer(m: PlainQwen2, i, x, cos, sin):
    """Pre-norm residual block in the order of tensorline/paged.py:245-276."""
    T = x.shape[0]
    h = rms_norm(x, m.layer(i, "input_layernorm.weight"), m.eps)
    q = linear(h, m.layer(i, "self_attn.q_proj.weight"), m.layer(i, "self_attn.q_proj.bias")).view(T, m.nq, m.d)
    k = linear(h, m.layer(i, "self_attn.k_proj.weight"), m.layer(i, "self_attn.k_proj.bias")).view(T, m.nkv, m.d)
    v = linear(h, m.layer(i, "self_attn.v_proj.weight"), m.layer(i, "self_attn.v_proj.bias")).view(T, m.nkv, m.d)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention(q, k, v, m.window[i]).reshape(T, m.nq * m.d)
    x = x + linear(o, m.layer(i, "self_attn.o_proj.weight"))
    h = rms_norm(x, m.layer(i, "post_attention_layernorm.weight"), m.eps)
    return x + swiglu(h, m.layer(i, "mlp.gate_proj.weight"), m.layer(i, "mlp.up_proj.weight"),
                      m.layer(i, "mlp.down_proj.weight"))


def forward(m: PlainQwen2, ids, rows=None) -> torch.Tensor:
    """Logits [T, V] (float64) at every position of one whole sequence
    (tensorline/paged.py:240-287 without the cache); `rows`: only these positions."""
    ids = list(ids)
    x = embedding(m.w["model.embed_tokens.weight"], ids)
    cos, sin = rope_cos_sin(range(len(ids)), m.d, m.theta)
    cos, sin = cos.to(x.dtype), sin.to(x.dtype)               # float64 unless the weights were narrowed
    for i in range(m.L):
        x = decoder_layer(m, i, x, cos, sin)
    if rows is not None:
        x = x[list(rows)]
    h = rms_norm(x, m.w["model.norm.weight"], m.eps)
    head = m.w["model.embed_tokens.weight"] if m.tied else m.w["lm_head.weight"]
    return linear(h, head)


def greedy_generate(m: PlainQwen2, prompt, n_new):
    """The one-request loop of tensorline/engine.py:86-115 with argmax sampling
    (engine.py:43-44); lowest index wins a tie."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(m, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out


# ---------------------------------------------------------------- sampling

def sampling_distribution(logits, temperature, top_p=1.0):
    """The distribution tensorline/engine.py:45-50 draws from: softmax(logits / T) in float,
    then (top_p < 1) sort descending, keep a token while the mass before it is < top_p,
    renormalise."""
    probs = torch.softmax(torch.as_tensor(logits, dtype=F64) / temperature, dim=-1)
    if top_p < 1.0:
        sp, idx = torch.sort(probs, descending=True, stable=True)
        keep = torch.cumsum(sp, dim=-1) - sp < top_p
        kept = torch.zeros_like(probs)
        kept[idx[keep]] = sp[keep]
        probs = kept / kept.sum()
    return probs


def inverse_cdf_pick(probs, u):
    """Index of the first token (in vocabulary order) whose cumulative mass exceeds u * total."""
    c = torch.cumsum(probs, dim=-1)
    i = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=c.dtype), right=True))
    return min(i, probs.numel() - 1)
