"""Plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, float32.

Written from the formulas of zeeshan8281/cloud-inference-from-scratch (each function cites
the file and lines it restates) and compared once with that project's own model code on
the CPU: ``tests/golden/make_golden.py`` wrote ``tests/golden/*.npz`` from
``cloud_engine.model.Qwen2CausalLM`` and ``tests/test_plain_model.py`` checks this file
against them.  It shares no code with the product package: it reads config.json and
model.safetensors itself and uses torch only for float32 arithmetic.

Two things go beyond the reference so that the engine's generality can be checked:
``window`` in ``attention`` (a query at position p sees keys p-window+1..p) and a run
``schedule`` in ``forward`` (a layer may run twice; a run may read the keys and values an
earlier run produced instead of its own).  Both default to the reference's behaviour.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


def read_model_folder(model_dir):
    """config.json as a dict and every tensor of model.safetensors as float32."""
    model_dir = Path(model_dir)
    with open(model_dir / "config.json", encoding="utf-8") as handle:
        config = json.load(handle)
    weights = {}
    for path in sorted(model_dir.glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in handle.keys():  # noqa: SIM118
                weights[name] = handle.get_tensor(name).to(torch.float32)
    return config, weights


def head_dim_of(config):
    # model.py:66-75: head_dim = hidden_size // num_attention_heads (explicit key wins here)
    return config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"]


def embedding(table, token_ids):
    """model.py:210 -- row gather, no scaling."""
    return table[torch.as_tensor(token_ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """attention.py:52-57 -- x * rsqrt(mean(x^2) + eps), then times the gain."""
    x = x.to(torch.float32)
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_tables(rotary_dim, positions, theta):
    """attention.py:60-67 -- inv_freq[j] = theta^(-2j/R); angles = pos * inv_freq; cat(ang, ang)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    angles = torch.as_tensor(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((angles, angles), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x):
    """attention.py:70-72."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x, cos, sin):
    """attention.py:75-85 -- x: [T, heads, D]; cos/sin: [T, R] with R <= D (rest passes through)."""
    rotary = cos.shape[-1]
    rotated = x[..., :rotary] * cos[:, None, :] + rotate_half(x[..., :rotary]) * sin[:, None, :]
    return torch.cat((rotated, x[..., rotary:]), dim=-1)


def linear(x, weight, bias=None):
    """nn.Linear as used in model.py:107-137: y = x W^T + b."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def attention(q, k, v, scale, window=0, positions=None):
    """attention.py:88-112 and 144-147 -- q: [T, Hq, D]; k, v: [T, Hkv, D]; causal softmax in
    float32; q head h reads kv head h // (Hq/Hkv).  Returns [T, Hq*D]."""
    tokens, num_heads, dim = q.shape
    group = num_heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    pos = torch.arange(tokens) if positions is None else torch.as_tensor(positions)
    allowed = pos[:, None] >= pos[None, :]
    if window > 0:
        allowed = allowed & (pos[:, None] - pos[None, :] < window)
    scores = scores.masked_fill(~allowed[None, :, :], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v).reshape(tokens, num_heads * dim)


def swiglu(x, gate, up, down):
    """model.py:99-100 -- down(silu(gate(x)) * up(x))."""
    return linear(torch.nn.functional.silu(linear(x, gate)) * linear(x, up), down)


def attention_layer(x, weights, prefix, config, positions, window=0, shared_kv=None):
    """model.py:132-137, 214-217 -- projections (+bias), rotary on q and k, attention, o_proj.
    Returns (update, (k, v)); with ``shared_kv`` the keys and values of another run are used."""
    heads = config["num_attention_heads"]
    kv_heads = config["num_key_value_heads"]
    dim = head_dim_of(config)
    tokens = x.shape[0]

    def bias(name):
        return weights.get(f"{prefix}{name}.bias")

    q = linear(x, weights[f"{prefix}q_proj.weight"], bias("q_proj")).view(tokens, heads, dim)
    cos, sin = rope_tables(dim, positions, config.get("rope_theta", 10000.0))
    q = apply_rope(q, cos, sin)
    if shared_kv is None:
        k = linear(x, weights[f"{prefix}k_proj.weight"], bias("k_proj")).view(tokens, kv_heads, dim)
        v = linear(x, weights[f"{prefix}v_proj.weight"], bias("v_proj")).view(tokens, kv_heads, dim)
        k = apply_rope(k, cos, sin)
    else:
        k, v = shared_kv
    mixed = attention(q, k, v, 1.0 / math.sqrt(dim), window=window, positions=positions)
    return linear(mixed, weights[f"{prefix}o_proj.weight"]), (k, v)


def decoder_layer(h, weights, index, config, positions, window=0, shared_kv=None):
    """model.py:212-220."""
    prefix = f"model.layers.{index}."
    eps = config["rms_norm_eps"]
    x = rms_norm(h, weights[prefix + "input_layernorm.weight"], eps)
    update, kv = attention_layer(x, weights, prefix + "self_attn.", config, positions, window, shared_kv)
    h = h + update
    x = rms_norm(h, weights[prefix + "post_attention_layernorm.weight"], eps)
    h = h + swiglu(
        x,
        weights[prefix + "mlp.gate_proj.weight"],
        weights[prefix + "mlp.up_proj.weight"],
        weights[prefix + "mlp.down_proj.weight"],
    )
    return h, kv


def lm_head(h, weights, config):
    """model.py:226-227 -- tied: the embedding matrix; else lm_head.weight; float32 product."""
    matrix = (
        weights["model.embed_tokens.weight"]
        if config["tie_word_embeddings"]
        else weights["lm_head.weight"]
    )
    return h.to(torch.float32) @ matrix.to(torch.float32).t()


def forward(config, weights, token_ids, schedule=None, window=0):
    """Logits [T, vocab] of one whole sequence starting at position 0 (model.py:194-228).

    ``schedule``: list of (layer index, index of the earlier run whose k/v to read, or None).
    ``window``: one window for every run, or a list with one window per run (0: all keys).
    """
    positions = list(range(len(token_ids)))
    h = embedding(weights["model.embed_tokens.weight"], token_ids)
    if schedule is None:
        schedule = [(index, None) for index in range(config["num_hidden_layers"])]
    produced = []
    windows = list(window) if isinstance(window, (list, tuple)) else [window] * len(schedule)
    for (layer, reads), run_window in zip(schedule, windows):
        shared = produced[reads] if reads is not None else None
        h, kv = decoder_layer(h, weights, layer, config, positions, run_window, shared)
        produced.append(kv)
    h = rms_norm(h, weights["model.norm.weight"], config["rms_norm_eps"])
    return lm_head(h, weights, config)


def greedy_generate(config, weights, prompt, steps, eos_token_id=None):
    """engine.py:486-488 with scheduler.py:593-607 -- argmax of the last row, append, repeat;
    stops after an EOS token (which is kept) or ``steps`` tokens."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        token = int(torch.argmax(forward(config, weights, tokens)[-1]).item())
        out.append(token)
        tokens.append(token)
        if eos_token_id is not None and token == eos_token_id:
            break
    return out


def temperature_probs(logits, temperature):
    """softmax(logits / T) in float32; the sampling rule itself is this framework's own."""
    return torch.softmax(logits.to(torch.float32) / temperature, dim=-1)
