"""A plain, slow implementation of the Qwen2 decoder: whole sequences, no cache.

This file is the oracle of the tests.  It shares no code with ``einf_b200``:
it reads ``config.json`` and ``model.safetensors`` itself and computes every
part with ordinary PyTorch on the CPU, one function per part, written from the
formulas of the reference (paths are relative to the reference project; each
function cites the lines it restates).  ``tests/golden/`` holds the outputs of
the reference's own model code on tiny random models, and
``tests/test_plain_vs_golden.py`` checks this file against them.

``rounding="bfloat16"`` rounds the activations to bfloat16 at the places where
a bfloat16 engine stores them (after every matrix product, norm, rotation,
attention and activation), keeping the arithmetic inside each part in 32-bit,
which is the numerical contract of the reference's kernels.  The residual
stream itself is never rounded: the engine keeps it in 32-bit.

The sliding window and an explicit layer order have no counterpart in the
reference (it reads no window key, ``src/einf/executors/torch/qwen.py:93-117``,
and runs layers 0..L-1, ``qwen.py:753-761``); they rest on their definitions:
query ``i`` sees keys ``j`` with ``i - window < j <= i``; the order is a list of
(layer, entry whose keys and values it reads instead of its own).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


# ---------------------------------------------------------------------------
# Reading a model folder
# ---------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors, upcast to ``dtype``.

    The reference reads ``model.safetensors`` with ``load_file`` and aliases
    ``lm_head.weight`` to the embedding when tied (``qwen.py:703-722``).
    """
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            tensor = handle.get_tensor(name)
            tensors[name] = tensor.to(dtype) if tensor.is_floating_point() else tensor
    if config["tie_word_embeddings"] and "lm_head.weight" not in tensors:
        tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"]
    return config, tensors


def head_size(config):
    """``hidden_size // num_attention_heads`` (``qwen.py:85-87``) unless given."""
    if config.get("head_dim") is not None:
        return config["head_dim"]
    return config["hidden_size"] // config["num_attention_heads"]


def window_of_layer(config, layer):
    if not config.get("use_sliding_window", False):
        return None
    first = config.get("max_window_layers")
    first = 0 if first is None else first
    return config["sliding_window"] if layer >= first else None


def _rounder(rounding):
    if rounding in (None, "float32"):
        return lambda x: x
    if rounding == "bfloat16":
        return lambda x: x.to(torch.bfloat16).to(x.dtype)
    raise ValueError(rounding)


# ---------------------------------------------------------------------------
# Parts
# ---------------------------------------------------------------------------
def embedding(token_ids, table):
    """``h0[t] = embed[token[t]]``, no scaling (``qwen.py:744``)."""
    return table[torch.as_tensor(token_ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """``w * x * rsqrt(mean(x^2) + eps)`` in 32-bit (``fused_ops.py:41-48``)."""
    variance = x.float().pow(2).mean(dim=-1, keepdim=True) if x.dtype != torch.float64 else x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_cos_sin(positions, dim, theta, dtype=torch.float32):
    """``inv_freq[i] = theta^(-2i/dim)``; angles ``pos * inv_freq`` repeated twice
    (``model_runner.py:42-60``)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=dtype) / dim))
    freqs = torch.as_tensor(positions, dtype=dtype)[:, None] * inv_freq[None, :]
    angles = torch.cat((freqs, freqs), dim=-1)
    return angles.cos()[:, None, :], angles.sin()[:, None, :]


def rotate_half(x):
    """``cat(-x2, x1)`` over the two halves of the head (``model_runner.py:63-66``)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x, cos, sin):
    """``x * cos + rotate_half(x) * sin`` (``model_runner.py:69-78``)."""
    return x * cos + rotate_half(x) * sin


def qkv_projection(x, tensors, prefix, num_heads, num_kv_heads, size, round_=lambda t: t):
    """Three linear layers with bias, viewed ``[T, heads, size]``
    (``packed_qkv.py:135-153``, ``qwen.py:384-387``)."""
    q = round_(x @ tensors[prefix + "q_proj.weight"].T) + tensors[prefix + "q_proj.bias"]
    k = round_(x @ tensors[prefix + "k_proj.weight"].T) + tensors[prefix + "k_proj.bias"]
    v = round_(x @ tensors[prefix + "v_proj.weight"].T) + tensors[prefix + "v_proj.bias"]
    tokens = x.shape[0]
    return (
        q.view(tokens, num_heads, size),
        k.view(tokens, num_kv_heads, size),
        v.view(tokens, num_kv_heads, size),
    )


def causal_attention(q, k, v, scale, window=None):
    """Softmax((Q K^T) * scale) V with a causal mask; query head ``h`` uses
    key/value head ``h // (Hq / Hkv)`` (``model_runner.py:125-151``,
    ``paged_attention_cuda.cu:71``; scale ``1/sqrt(D)`` at ``qwen.py:453,476,485``).
    ``q`` is ``[T, Hq, D]``, ``k`` and ``v`` ``[T, Hkv, D]``; the whole sequence
    is present, so query ``i`` sees keys ``j <= i`` (and ``j > i - window``)."""
    tokens, num_heads, _ = q.shape
    groups = num_heads // k.shape[1]
    k = k.repeat_interleave(groups, dim=1)
    v = v.repeat_interleave(groups, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(tokens)[:, None]
    j = torch.arange(tokens)[None, :]
    visible = j <= i
    if window is not None:
        visible &= j > i - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probabilities = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", probabilities, v)


def swiglu(x, gate_weight, up_weight, down_weight, round_=lambda t: t):
    """``down(silu(gate(x)) * up(x))`` (``qwen.py:209-212``; the packed form
    ``qwen.py:206-208`` with ``fused_ops.py:71-77`` is the same function)."""
    gate = round_(x @ gate_weight.T)
    up = round_(x @ up_weight.T)
    hidden = round_(torch.nn.functional.silu(gate) * up)
    return round_(hidden @ down_weight.T)


# ---------------------------------------------------------------------------
# The whole model
# ---------------------------------------------------------------------------
def attention_block(x, positions, config, tensors, layer, round_, shared_kv=None):
    """QKV with bias, rotation of Q and K, attention, output projection without
    bias (``qwen.py:374-489``).  Returns the output and the (K, V) it used."""
    prefix = f"model.layers.{layer}.self_attn."
    size = head_size(config)
    q, k, v = qkv_projection(
        x, tensors, prefix, config["num_attention_heads"], config["num_key_value_heads"], size, round_
    )
    v = round_(v)
    cos, sin = rope_cos_sin(positions, size, config["rope_theta"], dtype=x.dtype)
    q = round_(apply_rope(q, cos, sin))
    k = round_(apply_rope(k, cos, sin))
    if shared_kv is not None:
        k, v = shared_kv
    out = causal_attention(q, k, v, 1.0 / math.sqrt(size), window_of_layer(config, layer))
    out = round_(out).reshape(x.shape[0], -1)
    return round_(out @ tensors[prefix + "o_proj.weight"].T), (k, v)


def forward(config, tensors, token_ids, schedule=None, rounding=None, return_hidden=False, rows=None):
    """Logits ``[T, vocab]`` of one whole sequence from position 0 (with ``rows``, a list of
    positions, only those rows of the output matrix product are computed: ``[len(rows), vocab]``).

    Pre-norm residual stream (``qwen.py:526-563``): ``h += attn(norm1(h))``,
    ``h += mlp(norm2(h))``; final norm and the output matrix
    (``qwen.py:762-773``).  ``schedule`` is a list of ``(layer, cache_from)``;
    by default layers 0..L-1, each with keys and values of its own.
    """
    round_ = _rounder(rounding)
    eps = config["rms_norm_eps"]
    if schedule is None:
        schedule = [(layer, None) for layer in range(config["num_hidden_layers"])]
    positions = torch.arange(len(token_ids))
    hidden = embedding(token_ids, tensors["model.embed_tokens.weight"])
    kv_of_entry = []
    for layer, cache_from in schedule:
        prefix = f"model.layers.{layer}."
        x = round_(rms_norm(hidden, tensors[prefix + "input_layernorm.weight"], eps))
        shared = kv_of_entry[cache_from] if cache_from is not None else None
        mixed, kv = attention_block(x, positions, config, tensors, layer, round_, shared)
        kv_of_entry.append(kv)
        hidden = hidden + mixed
        x = round_(rms_norm(hidden, tensors[prefix + "post_attention_layernorm.weight"], eps))
        hidden = hidden + swiglu(
            x,
            tensors[prefix + "mlp.gate_proj.weight"],
            tensors[prefix + "mlp.up_proj.weight"],
            tensors[prefix + "mlp.down_proj.weight"],
            round_,
        )
    final = round_(rms_norm(hidden, tensors["model.norm.weight"], eps))
    if rows is not None:
        final = final[torch.as_tensor(list(rows), dtype=torch.long)]
    logits = final @ tensors["lm_head.weight"].T
    if return_hidden:
        return logits, final
    return logits


# ---------------------------------------------------------------------------
# Sampling
# ---------------------------------------------------------------------------
_MASK64 = (1 << 64) - 1


def uniform_from_key(seed, sample_index):
    """The engine's counter-based uniform number in [0, 1): two rounds of the
    splitmix64 finaliser over ``seed`` and ``sample_index``, top 24 bits.

    The reference seeds a fresh generator with ``seed + sample_index`` for each
    sampled token (``sampler.py:93-94``) so that a request's stream does not
    depend on the batch; the generator itself is ours.
    """
    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)

    z = mix(seed & _MASK64)
    z = mix(z ^ (sample_index & _MASK64))
    return (z >> 40) / float(1 << 24)


def filtered_probabilities(logits, temperature, top_k=None, top_p=1.0, min_p=0.0):
    """The distribution the reference samples from (``sampler.py:43-88``):
    logits / T, keep the k largest, keep the smallest prefix of the sorted
    probabilities whose mass reaches ``top_p`` (the crossing token included),
    drop tokens below ``min_p`` times the largest probability, renormalise."""
    logits = logits.float() / temperature
    if top_k is not None and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.numel())).values[-1]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, order = torch.sort(logits, descending=True)
        cumulative = torch.softmax(sorted_logits, dim=-1).cumsum(-1)
        remove = cumulative > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        sorted_logits = sorted_logits.masked_fill(remove, float("-inf"))
        logits = torch.empty_like(logits).scatter(0, order, sorted_logits)
    if min_p > 0.0:
        probabilities = torch.softmax(logits, dim=-1)
        logits = logits.masked_fill(probabilities < probabilities.max() * min_p, float("-inf"))
    return torch.softmax(logits, dim=-1)


def sample_token(logits, temperature, seed=0, sample_index=0, top_k=None, top_p=1.0, min_p=0.0):
    """Greedy for temperature 0 (first largest index, ``sampler.py:31-32``); else
    the inverse of the cumulative distribution at the keyed uniform number."""
    if temperature == 0:
        return int(torch.argmax(logits.float()))
    probabilities = filtered_probabilities(logits, temperature, top_k, top_p, min_p)
    u = uniform_from_key(seed, sample_index)
    cumulative = probabilities.double().cumsum(-1)
    target = u * float(cumulative[-1])
    index = int(torch.searchsorted(cumulative, torch.tensor(target, dtype=torch.float64), right=True))
    return min(index, logits.numel() - 1)


def greedy_generate(config, tensors, prompt, steps, rounding=None):
    """Recompute the whole sequence for each new token; argmax of the last row."""
    tokens = list(prompt)
    for _ in range(steps):
        logits = forward(config, tensors, tokens, rounding=rounding)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]
