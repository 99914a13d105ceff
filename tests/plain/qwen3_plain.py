"""A plain, slow implementation of the dense Qwen3 decoder for whole sequences.

Written from the reference's formulas, one function per part, each citing the
lines it restates.  It has no cache, no batching and no kernels, runs on the CPU
in PyTorch, and shares no code with the engine: tests compare the engine to it.
``tests/golden/make_golden.py`` compared it once against the reference's own
``qil.model.Qwen3`` on a tiny random model; the stored outputs are in
``tests/golden/``.

Weights are a dict of tensors under checkpoint names; ``cfg`` is the parsed
config.json (a dict).  ``dtype`` is the activation dtype: float32 for the exact
path, bfloat16 to follow the rounding points of a bfloat16 run.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """qil/model.py:21-23: float32 statistics and scaling, cast back, then times weight."""
    x32 = x.float()
    normalized = x32 * (x32.square().mean(dim=-1, keepdim=True) + eps).rsqrt()
    return normalized.to(x.dtype) * weight.to(x.dtype)


def rotary_angles(positions, head_dim, theta):
    """qil/model.py:103-108: inverse frequencies in float32 on the CPU, angle = position * frequency."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    return positions.float()[:, None] * inv_freq[None, :]


def rotate(x, angles):
    """qil/model.py:42-46: half-split rotation; cos and sin rounded to x's dtype. x [T, heads, D]."""
    cosine, sine = angles.cos().to(x.dtype)[:, None], angles.sin().to(x.dtype)[:, None]
    left, right = x.chunk(2, dim=-1)
    return torch.cat((left * cosine - right * sine, left * sine + right * cosine), dim=-1)


def linear(x, weight, bias=None):
    """qil/model.py:32-40: nn.Linear, weight [out, in]."""
    y = x @ weight.to(x.dtype).t()
    if bias is not None:
        y = y + bias.to(x.dtype)
    return y


def causal_attention(q, k, v, scale, window=0):
    """qil/model.py:59-68: GQA by repeating kv heads, mask key j <= query position, softmax, times v.

    q [T, Hq, D], k and v [T, Hkv, D] for positions 0..T-1.  Scores and softmax in
    float32; the result is cast to q's dtype.  ``window`` > 0 also masks keys more than
    window-1 positions back (not used by the reference; for parts tests).
    """
    T, n_q, _ = q.shape
    group = n_q // k.shape[1]
    k = k.repeat_interleave(group, dim=1).transpose(0, 1).float()      # [Hq, T, D]
    v = v.repeat_interleave(group, dim=1).transpose(0, 1).float()
    scores = torch.einsum("thd,hjd->htj", q.float(), k) * scale
    pos = torch.arange(T)
    mask = pos[None, :] <= pos[:, None]
    if window > 0:
        mask &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~mask[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("htj,hjd->thd", probs, v)
    return out.to(q.dtype)


def attention_block(x, w, prefix, cfg, angles):
    """qil/model.py:51-69 without the cache: projections, per-head q/k norm, rotation, attention, o_proj."""
    T = x.shape[0]
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg.get("rms_norm_eps", 1e-6)
    bias = (lambda name: w.get(prefix + f"self_attn.{name}.bias"))
    q = linear(x, w[prefix + "self_attn.q_proj.weight"], bias("q_proj")).reshape(T, n_q, d)
    k = linear(x, w[prefix + "self_attn.k_proj.weight"], bias("k_proj")).reshape(T, n_kv, d)
    v = linear(x, w[prefix + "self_attn.v_proj.weight"], bias("v_proj")).reshape(T, n_kv, d)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q, k = rotate(q, angles), rotate(k, angles)
    attended = causal_attention(q, k, v, d ** -0.5).reshape(T, n_q * d)
    return linear(attended, w[prefix + "self_attn.o_proj.weight"], bias("o_proj"))


def gated_mlp(x, w, prefix):
    """qil/model.py:71: contract(silu(gate(n)) * expand(n))."""
    gate = torch.nn.functional.silu(linear(x, w[prefix + "mlp.gate_proj.weight"]))
    up = linear(x, w[prefix + "mlp.up_proj.weight"])
    return linear(gate * up, w[prefix + "mlp.down_proj.weight"])


def decoder_block(x, w, prefix, cfg, angles):
    """qil/model.py:48-71: x + attn(norm(x)); then x + mlp(norm(x))."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    x = x + attention_block(rms_norm(x, w[prefix + "input_layernorm.weight"], eps), w, prefix, cfg, angles)
    return x + gated_mlp(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps), w, prefix)


def logits(tokens, w, cfg, dtype=torch.float32):
    """qil/model.py:110-134 with logits_mode='all': float32 logits [T, vocab] of a whole sequence."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    angles = rotary_angles(torch.arange(len(tokens)), cfg["head_dim"], cfg.get("rope_theta", 1e6))
    x = w["model.embed_tokens.weight"].to(dtype)[tokens]
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_block(x, w, f"model.layers.{i}.", cfg, angles)
    x = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return linear(x, head).float()


def greedy(prompt, new_tokens, w, cfg, dtype=torch.float32, eos=()):
    """qil/engine.py:96-113: argmax of the last position, appended, until length or an eos token."""
    tokens, out = list(prompt), []
    for _ in range(new_tokens):
        token = int(logits(tokens, w, cfg, dtype)[-1].argmax())
        out.append(token)
        tokens.append(token)
        if token in eos:
            break
    return out


def gumbel_uniform(seed, counter, index):
    """The sampler's noise: uniform in (0,1) from (seed, draw counter, vocabulary index)."""
    mask = (1 << 64) - 1
    z = (seed ^ ((0x9E3779B97F4A7C15 * (counter + 1)) & mask)) & mask
    z = (z + index * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 30; z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27; z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return ((z >> 40) + 0.5) / 16777216.0


def sample(logit_row, temperature, seed, counter):
    """argmax(logit / T + Gumbel noise): a draw from softmax(logit / T); greedy when T == 0."""
    if temperature <= 0:
        return int(torch.as_tensor(logit_row).argmax())
    best, best_key = 0, -math.inf
    for i, value in enumerate(torch.as_tensor(logit_row).tolist()):
        u = gumbel_uniform(seed, counter, i)
        key = value / temperature - math.log(-math.log(u))
        if key > best_key:
            best, best_key = i, key
    return best
