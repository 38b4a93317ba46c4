"""Plain PyTorch statements of the engine's kernels, one function per kernel,
with the signatures of ``einf_b200.ops``.

Two uses.  The ``-m gpu`` tests run each kernel alone against its function here.
And :func:`emulate_kernels` swaps them in for the kernels, which lets the
engine's host logic (batch packing, cache, replay, scheduler and executor) be
tested on a machine without a GPU; the product itself has no such path.

Arithmetic is 32-bit (or 64-bit with ``HIGH_PRECISION``); results are rounded
once into the output's dtype, as the kernels do.
"""
from __future__ import annotations

import contextlib

import torch

_MASK64 = (1 << 64) - 1


def embed(tokens, table, residual, status):
    residual.copy_(table[tokens.long()].float())


def add_rmsnorm(x, residual, weight, eps, out, rows=None, status=None):
    total = residual.float()
    if x is not None:
        xf = x.float()
        if xf.dim() == 3:
            xf = xf.sum(0)
        total = total + xf
    source = total if rows is None else total[rows.long()]
    variance = source.pow(2).mean(-1, keepdim=True)
    out.copy_((weight * (source * torch.rsqrt(variance + eps))).to(out.dtype))
    if rows is None and x is not None:
        residual.copy_(total)


def rope_kv_write(qkv, bias, positions, inv_freq, slots, q_out, k_cache, v_cache,
                  num_heads, num_kv_heads, head_size, status):
    values = qkv.float()
    if values.dim() == 3:
        values = values.sum(0)
    tokens = values.shape[0]
    if bias is not None:
        values = values + bias
    q, k, v = values.split([num_heads * head_size, num_kv_heads * head_size, num_kv_heads * head_size], dim=-1)
    q = q.reshape(tokens, num_heads, head_size)
    k = k.reshape(tokens, num_kv_heads, head_size)
    v = v.reshape(tokens, num_kv_heads, head_size)
    half = inv_freq.shape[0]
    if half:
        angles = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]

        def rotate(x):
            a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)

        q, k = rotate(q), rotate(k)
    q_out.copy_(q.reshape(q_out.shape).to(q_out.dtype))
    if slots is not None:
        page_size = k_cache.shape[2]
        keep = slots >= 0
        page = (slots[keep] // page_size).long()
        offset = (slots[keep] % page_size).long()
        k_cache[page, :, offset, :] = k[keep].to(k_cache.dtype)
        v_cache[page, :, offset, :] = v[keep].to(v_cache.dtype)


def silu_mul(gate_up, out):
    inter = out.shape[-1]
    gate_up = gate_up.float()
    if gate_up.dim() == 3:
        gate_up = gate_up.sum(0)
    g, u = gate_up[:, :inter], gate_up[:, inter:]
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def linear(x, weight, bias, out):
    result = x.float() @ weight.float().T
    if bias is not None:
        result = result + bias
    out.copy_(result.to(out.dtype))


def gemm_simt(x, weight, bias, out):
    linear(x, weight, bias, out)


def project(x, weight, status, out_dtype=None, allow_partial=True):
    out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
    linear(x, weight, None, out)
    return out


def paged_attention_generic(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window, status):
    tokens, num_heads, head_size = q.shape
    _, num_kv_heads, page_size, _ = k_cache.shape
    groups = num_heads // num_kv_heads
    for t in range(tokens):
        r = int(seq_of_token[t])
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        keys = torch.arange(lo, pos + 1, device=q.device)
        pages = block_table[r, (keys // page_size).long()].long()
        offsets = (keys % page_size).long()
        k = k_cache[pages, :, offsets, :].float()      # [n, kv_heads, D]
        v = v_cache[pages, :, offsets, :].float()
        k = k.repeat_interleave(groups, dim=1)
        v = v.repeat_interleave(groups, dim=1)
        scores = torch.einsum("hd,nhd->hn", q[t].float(), k) * scale
        probabilities = torch.softmax(scores, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", probabilities, v).to(out.dtype)


def argmax(logits, tokens):
    tokens[: logits.shape[0]] = torch.argmax(logits, dim=-1).to(torch.int32)


def keyed_uniform(seed, index):
    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)

    z = mix(int(seed) & _MASK64)
    z = mix(z ^ (int(index) & _MASK64))
    return (z >> 40) / float(1 << 24)


def kept_weights(row, temperature, top_k, top_p, min_p):
    """Unnormalised probabilities of the tokens a row may draw (0 for dropped ones).  Tokens with
    equal scaled logits stay or go together: top-k keeps every token that ties the k-th, top-p
    keeps a token iff the mass of the strictly more probable ones has not passed top_p of the
    mass.  (The reference sorts, so among equal logits it keeps whichever the sort puts first.)"""
    scaled = row.float() / temperature
    weights = torch.exp(scaled - scaled.max())
    keep = torch.ones_like(weights, dtype=torch.bool)
    if top_k and top_k < row.numel():
        kth = torch.topk(scaled, top_k).values[-1]
        keep &= scaled >= kth
    if top_p < 1.0:
        masked = torch.where(keep, weights, torch.zeros_like(weights)).double()
        values, which = torch.unique(scaled, return_inverse=True)               # ascending
        mass_of_value = torch.zeros(values.numel(), dtype=torch.float64).index_add_(0, which, masked)
        above = mass_of_value.flip(0).cumsum(0).flip(0) - mass_of_value         # mass of the strictly larger values
        keep &= (above <= top_p * masked.sum())[which]
    if min_p > 0.0:
        keep &= weights >= min_p
    return torch.where(keep, weights, torch.zeros_like(weights))


def sample(logits, tokens, temperature, top_k, top_p, min_p, seed, sample_index):
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        if t <= 0:
            tokens[r] = int(torch.argmax(logits[r]))
            continue
        weights = kept_weights(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r])).double()
        cumulative = weights.cumsum(0)
        target = keyed_uniform(int(seed[r]), int(sample_index[r])) * float(cumulative[-1])
        index = int(torch.searchsorted(cumulative, torch.tensor(target, dtype=torch.float64), right=True))
        tokens[r] = min(index, logits.shape[1] - 1)


def advance_decode(token_ids, positions, context_lens, sampled, slots, block_tables, page_size):
    n = sampled.shape[0]
    token_ids[:n] = sampled
    positions[:n] += 1
    context_lens[:n] += 1
    for slot, table in zip(slots, block_tables):
        for i in range(n):
            if int(slot[i]) < 0:
                continue
            position = int(positions[i])
            slot[i] = int(table[i, position // page_size]) * page_size + position % page_size


def zero_fresh_state(state, state_slots, q_start, positions):
    for request in range(state_slots.shape[0]):
        slot = int(state_slots[request])
        if 0 <= slot < state.shape[0] and int(positions[int(q_start[request])]) == 0:
            state[slot] = 0


def has_fast_attention(dtype, head_size):
    return False          # the plain statement of attention serves every dtype here


def report(tokens, count, status, host):
    host[:count] = tokens[:count]
    host[count] = status[0]


def ensure_built(names):
    return None


_NAMES = (
    "embed", "add_rmsnorm", "rope_kv_write", "silu_mul", "linear", "gemm_simt", "project",
    "paged_attention_generic", "argmax", "sample", "ensure_built", "advance_decode", "report",
    "zero_fresh_state", "has_fast_attention",
)


@contextlib.contextmanager
def emulate_kernels():
    """Within the block, ``einf_b200.ops`` computes with the functions above and a
    ``ModelRunner`` accepts the CPU device."""
    from einf_b200 import ops
    from einf_b200.engine.runner import ModelRunner

    saved_ops = {name: getattr(ops, name) for name in _NAMES}
    saved = tuple(ModelRunner.__dict__[n] for n in ("_check_device", "_guard", "synchronize", "_graphable"))
    for name in _NAMES:
        setattr(ops, name, globals()[name])
    ModelRunner._check_device = staticmethod(lambda device: None)
    ModelRunner._guard = lambda self: contextlib.nullcontext()
    ModelRunner.synchronize = lambda self: None
    ModelRunner._graphable = staticmethod(lambda requests: False)   # no CUDA graphs without CUDA
    try:
        yield
    finally:
        for name, function in saved_ops.items():
            setattr(ops, name, function)
        ModelRunner._check_device, ModelRunner._guard, ModelRunner.synchronize, ModelRunner._graphable = saved
