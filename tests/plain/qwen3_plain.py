"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

Written from the reference's formulas (each function cites the file and lines
under the reference project); it shares no code with ``enginekernel_b200``: it has
its own config reader, its own safetensors reader and uses only elementary torch
operations.  It was compared once with the reference's own model code on the CPU;
``tests/golden/make_golden.py`` is the script and ``tests/golden/*.pt`` are the
outputs, which ``tests/test_plain.py`` replays.

Everything runs in the dtype of the tensors it is given.  In float32 nothing is
rounded.  In bfloat16 every elementary operation rounds, which reproduces the
reference's rounding points (normalise in 32-bit, round, then multiply by the gain,
and so on).
"""

from __future__ import annotations

import glob
import json
import math
import os

import torch


# --------------------------------------------------------------------------- loading
def read_config(folder):
    """engine/ek_model.py:26-42 - keys and defaults."""
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    cfg = {
        "hidden_size": raw["hidden_size"],
        "num_layers": raw["num_hidden_layers"],
        "num_heads": raw["num_attention_heads"],
        "num_kv_heads": raw["num_key_value_heads"],
        "intermediate_size": raw["intermediate_size"],
        "vocab_size": raw["vocab_size"],
        "rms_eps": raw.get("rms_norm_eps", 1e-6),
        "rope_theta": raw.get("rope_theta", 10000.0),
        "tie": raw.get("tie_word_embeddings", False),
        "max_position": raw.get("max_position_embeddings", 32768),
    }
    cfg["head_dim"] = raw.get("head_dim", cfg["hidden_size"] // cfg["num_heads"])
    return cfg


def read_weights(folder, dtype):
    """engine/ek_model.py:117-160 - tensors by checkpoint name, cast on read.  The
    reference concatenates q/k/v and gate/up; here they stay separate matrices."""
    from safetensors import safe_open
    out = {}
    for fn in sorted(glob.glob(os.path.join(folder, "*.safetensors"))):
        with safe_open(fn, framework="pt", device="cpu") as f:
            for k in f.keys():
                out[k] = f.get_tensor(k).to(dtype)
    return out


class PlainModel:
    def __init__(self, folder, dtype=torch.float32):
        self.cfg = read_config(folder)
        self.w = read_weights(folder, dtype)
        self.dtype = dtype
        if self.cfg["tie"]:                                   # engine/ek_model.py:134
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]


# --------------------------------------------------------------------------- parts
def rms_norm(x, gain, eps):
    """engine/ek_kernels.py:1025-1028 (and 98-103): mean of squares and scaling in
    32-bit, the result rounded to the model dtype, then multiplied by the gain."""
    xf = x.float()
    xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return gain * xn.to(x.dtype)


def rope_tables(num_positions, head_dim, theta, dtype):
    """engine/ek_model.py:164-174: inverse frequencies theta^(-2j/D), angles
    position x frequency, the half table repeated twice (NeoX pairing), computed in
    32-bit and stored in the model dtype."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(num_positions, dtype=torch.float32)
    freqs = torch.outer(t, inv)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x):
    """engine/ek_kernels.py:1129: cat(-x[D/2:], x[:D/2])."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def qk_norm_rope(x, gain, cos, sin, eps):
    """engine/ek_kernels.py:1126-1130: per-head RMSNorm over the head dimension,
    then x*cos + rotate_half(x)*sin.  x: [S, heads, D]; cos/sin: [S, D]."""
    xn = rms_norm(x, gain, eps)
    return xn * cos.unsqueeze(1) + rotate_half(xn) * sin.unsqueeze(1)


def causal_gqa_attention(q, k, v, scale, window=None):
    """engine/ek_model.py:475-488 (the decode formula applied at every position):
    query head h reads key/value head h // G; scores in 32-bit times ``scale``;
    keys after the query are masked with -inf; softmax in 32-bit, cast to the value
    dtype, and the weighted sum of values in 32-bit.
    q: [S, NH, D]; k, v: [S, NKV, D] -> [S, NH*D].  ``window`` (not used by Qwen3,
    kept for tests of the attention part alone) hides keys further back than
    ``window - 1`` positions."""
    s, nh, d = q.shape
    rep = nh // k.shape[1]
    kk = k.repeat_interleave(rep, 1)
    vv = v.repeat_interleave(rep, 1)
    scores = torch.einsum("thd,jhd->htj", q.float(), kk.float()) * scale
    i = torch.arange(s)
    hidden = i[None, :] > i[:, None]
    if window is not None:
        hidden = hidden | (i[None, :] <= i[:, None] - window)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(scores, dim=-1).to(v.dtype)
    o = torch.einsum("htj,jhd->thd", p.float(), vv.float()).to(q.dtype)
    return o.reshape(s, nh * d)


def attention_block(x, w, prefix, cfg, cos, sin):
    """engine/ek_model.py:298-311: q/k/v projections without bias, q/k norm and
    rotation, attention, output projection."""
    s = x.shape[0]
    nh, nkv, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].t()).view(s, nh, d)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].t()).view(s, nkv, d)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].t()).view(s, nkv, d)
    q = qk_norm_rope(q, w[prefix + "self_attn.q_norm.weight"], cos, sin, cfg["rms_eps"])
    k = qk_norm_rope(k, w[prefix + "self_attn.k_norm.weight"], cos, sin, cfg["rms_eps"])
    o = causal_gqa_attention(q, k, v, d ** -0.5)              # scale: engine/ek_model.py:71
    return o @ w[prefix + "self_attn.o_proj.weight"].t()


def swiglu_mlp(x, w, prefix):
    """engine/ek_model.py:205-209 with engine/ek_kernels.py:1062-1066:
    down(silu(gate(x)) * up(x))."""
    g = x @ w[prefix + "mlp.gate_proj.weight"].t()
    u = x @ w[prefix + "mlp.up_proj.weight"].t()
    return (torch.nn.functional.silu(g) * u) @ w[prefix + "mlp.down_proj.weight"].t()


def embed(ids, w):
    """engine/ek_model.py:290 - a row lookup, no scaling."""
    return w["model.embed_tokens.weight"][torch.as_tensor(ids, dtype=torch.long)]


def lm_head(h, w):
    """engine/ek_model.py:490-493."""
    return h @ w["lm_head.weight"].t()


# --------------------------------------------------------------------------- model
def hidden_states(model, ids):
    """engine/ek_model.py:291-334: residual wiring of the pre-norm blocks and the
    final norm.  Returns the normalised hidden state at every position [S, H]."""
    cfg, w = model.cfg, model.w
    s = len(ids)
    cos, sin = rope_tables(s, cfg["head_dim"], cfg["rope_theta"], model.dtype)
    r = embed(ids, w)
    for i in range(cfg["num_layers"]):
        p = f"model.layers.{i}."
        a = rms_norm(r, w[p + "input_layernorm.weight"], cfg["rms_eps"])
        r = r + attention_block(a, w, p, cfg, cos, sin)
        m = rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_eps"])
        r = r + swiglu_mlp(m, w, p)
    return rms_norm(r, w["model.norm.weight"], cfg["rms_eps"])


def logits(model, ids):
    """Logits at every position of one whole sequence, [S, V], in 32-bit."""
    return lm_head(hidden_states(model, ids), model.w).float()


def greedy(model, prompt, n):
    """engine/ek_model.py:490-493: arg-max, ties to the lowest index; the whole
    sequence is recomputed for every token."""
    ids = list(prompt)
    out = []
    for _ in range(n):
        t = int(torch.argmax(logits(model, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out


# --------------------------------------------------------------------------- sampling
_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key):
    """Philox-4x32 with 10 rounds on Python integers; counter 4 words, key 2 words."""
    c = list(counter)
    k = list(key)
    for _ in range(10):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed, stream, step, index):
    """The uniform number in (0, 1) that belongs to vocabulary entry ``index`` of the
    draw ``step`` of sequence ``stream`` under ``seed``: word index % 4 of the Philox
    block with counter (index // 4, step, stream, 0) and key (seed low, seed high);
    its top 23 bits b give (b + 0.5) / 2^23, which 32-bit floats hold exactly."""
    words = philox4x32((index // 4, step & 0xFFFFFFFF, stream & 0xFFFFFFFF, 0),
                       (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return ((words[index % 4] >> 9) + 0.5) / 8388608.0


def sample_token(logits_row, temperature, top_k, seed, stream, step):
    """Temperature / top-k sampling by the Gumbel-max rule: the drawn token is
    argmax_i(logit_i / temperature - log(-log(u_i))) over the ``top_k`` largest logits
    (all when 0; ties at the k-th value are all kept).  temperature 0 is arg-max."""
    row = logits_row.double()
    if temperature == 0:
        return int(torch.argmax(row))
    v = row.numel()
    keep = torch.ones(v, dtype=torch.bool)
    if top_k and top_k < v:
        kth = torch.topk(row, top_k).values[-1]
        keep = row >= kth
    best, best_score = -1, -math.inf
    for i in range(v):
        if not keep[i]:
            continue
        u = uniform_for(seed, stream, step, i)
        score = float(row[i]) / temperature - math.log(-math.log(u))
        if score > best_score:
            best, best_score = i, score
    return best
