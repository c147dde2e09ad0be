"""The reference's CPU PyTorch decode path, restated.  TEST INFRASTRUCTURE ONLY.

These are the functions the reference executes when no GPU backend applies;
the benchmark times them on the host cores as the CPU baseline ("port"), and
the tests use them as a second, float32 checker beside the C oracle.

Parity status: pinned - compared with the reference's own functions on seeded
inputs by ``tests/golden/make_golden.py`` (fixtures committed beside it).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def dense_decode(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """Exact decode as the reference's CPU path computes it.

    Follows ``stream_attention/gate1.py:157-183`` (``dense_attention_forward``,
    reached from ``decode.py:192-215`` for CPU tensors): BNHD inputs are
    brought to head-major, KV heads are expanded to the query head count with
    ``repeat_interleave`` and one non-causal SDPA call produces the result.
    query [B,1,Hq,D], key/value [B,N,Hkv,D]; returns [B,1,Hq,D].
    """

    q = query.transpose(1, 2).contiguous()
    k = key.transpose(1, 2).contiguous()
    v = value.transpose(1, 2).contiguous()
    q_heads, kv_heads = q.shape[1], k.shape[1]
    if q_heads != kv_heads:
        if q_heads % kv_heads:
            raise ValueError("query heads must be a multiple of KV heads")
        rep = q_heads // kv_heads
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    out = F.scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False)
    return out.transpose(1, 2).contiguous()


def paged_decode(
    query: torch.Tensor,
    key_pages: torch.Tensor,
    value_pages: torch.Tensor,
    page_table: torch.Tensor,
    lengths: torch.Tensor,
    *,
    layout: str = "NHD",
) -> torch.Tensor:
    """Page-streaming exact decode, one online-softmax update per page.

    Follows ``stream_attention/paged.py:201-256`` (``paged_exact_reference``):
    for every (row, query head) walk the row's active logical pages in order,
    look the physical page up in ``page_table``, clip the last page to the
    row length and fold the page into a running (max, denominator, numerator).
    """

    layout = layout.upper()
    batch, _, heads, dim = (int(x) for x in query.shape)
    if layout == "NHD":
        page_size, kv_heads = int(key_pages.shape[1]), int(key_pages.shape[2])
    else:
        kv_heads, page_size = int(key_pages.shape[1]), int(key_pages.shape[2])
    group = heads // kv_heads
    scale = 1.0 / math.sqrt(float(dim))
    out = torch.empty_like(query)
    for b in range(batch):
        n = int(lengths[b])
        pages = -(-n // page_size)
        for h in range(heads):
            kvh = h // group
            q = query[b, 0, h].float()
            m = torch.tensor(float("-inf"))
            den = torch.zeros(())
            num = torch.zeros(dim)
            for lp in range(pages):
                pp = int(page_table[b, lp])
                valid = min(page_size, n - lp * page_size)
                if layout == "NHD":
                    kp = key_pages[pp, :valid, kvh]
                    vp = value_pages[pp, :valid, kvh]
                else:
                    kp = key_pages[pp, kvh, :valid]
                    vp = value_pages[pp, kvh, :valid]
                s = (kp.float() @ q) * scale
                new_m = torch.maximum(m, s.max())
                corr = torch.exp(m - new_m)
                p = torch.exp(s - new_m)
                num = num * corr + (p[:, None] * vp.float()).sum(dim=0)
                den = den * corr + p.sum()
                m = new_m
            out[b, 0, h] = (num / den).to(out.dtype)
    return out


def seed_decode(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    tokens: torch.Tensor,
) -> torch.Tensor:
    """Seed-only decode: exact attention restricted to a fixed token set.

    Follows ``benchmarks/profile_seed_only_route_bundle_decode.py:450-507``
    (float32 scores, softmax and value accumulation over the gathered seed
    tokens, GQA map ``kv_head = head // group``).  BNHD inputs as elsewhere in
    this module: query [B,1,Hq,D], key/value [B,N,Hkv,D]; returns [B,1,Hq,D].
    """

    batch, _, heads, dim = (int(x) for x in query.shape)
    kv_heads = int(key.shape[2])
    group = heads // kv_heads
    if tokens.numel() == 0:
        return torch.zeros_like(query)
    idx = tokens.to(torch.long)
    k_sel = key.index_select(1, idx).float()      # [B,S,Hkv,D]
    v_sel = value.index_select(1, idx).float()
    kv_of_q = torch.arange(heads) // group
    k_q = k_sel.index_select(2, kv_of_q)          # [B,S,Hq,D]
    v_q = v_sel.index_select(2, kv_of_q)
    q = query[:, 0].float()                       # [B,Hq,D]
    scores = torch.einsum("bhd,bshd->bhs", q, k_q) / math.sqrt(float(dim))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("bhs,bshd->bhd", probs, v_q)
    return out[:, None].to(query.dtype)


def qwen_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x`` [B, H, 1, D] with ``cos``/``sin`` [B, 1, D], in the tensors' dtype.

    Follows ``benchmarks/profile_seed_only_fused_rope_parity.py:24-30`` (``_rotate_half`` /
    ``_apply_qwen_rope``): ``x * cos + concat(-x[D/2:], x[:D/2]) * sin``; every product and the sum
    are rounded to the dtype, as torch does for half-precision tensors.
    """

    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos.unsqueeze(1)) + (rotated * sin.unsqueeze(1))


def rope_append(q_raw, k_raw, v_raw, cos, sin, key_cache, value_cache, positions):
    """The reference's safe path for one decode step's cache update (same file, lines 92-102).

    q_raw [B,Hq,1,D], k_raw/v_raw [B,Hkv,1,D], cos/sin [B or 1,1,D] (None: no rotation), caches
    [B,Hkv,N,D] (updated in place), ``positions`` one int per row.  Returns the rotated query.
    """

    batch = k_raw.shape[0]
    if cos is not None:
        cos_b = cos.expand(batch, -1, -1)
        sin_b = sin.expand(batch, -1, -1)
        q_rot = qwen_rope(q_raw, cos_b, sin_b) if q_raw is not None else None
        k_rot = qwen_rope(k_raw, cos_b, sin_b)
    else:
        q_rot, k_rot = q_raw, k_raw
    for b, pos in enumerate(positions):
        key_cache[b, :, pos : pos + 1, :].copy_(k_rot[b])
        value_cache[b, :, pos : pos + 1, :].copy_(v_raw[b])
    return q_rot


def paged_rope_append(q_raw, k_raw, v_raw, cos, sin, key_pages, value_pages, page_table, positions, *, layout="NHD"):
    """Same update for a paged cache: row b goes to slot ``pos % page`` of ``page_table[b][pos // page]``.

    The reference has no paged writer; the addressing is that of its paged reader
    (``stream_attention/paged.py:217-255``).  Pages [P,page,Hkv,D] (NHD) or [P,Hkv,page,D] (HND),
    updated in place.
    """

    layout = layout.upper()
    page_size = key_pages.shape[1] if layout == "NHD" else key_pages.shape[2]
    batch = k_raw.shape[0]
    if cos is not None:
        cos_b = cos.expand(batch, -1, -1)
        sin_b = sin.expand(batch, -1, -1)
        q_rot = qwen_rope(q_raw, cos_b, sin_b) if q_raw is not None else None
        k_rot = qwen_rope(k_raw, cos_b, sin_b)
    else:
        q_rot, k_rot = q_raw, k_raw
    for b, pos in enumerate(positions):
        page = int(page_table[b, pos // page_size])
        slot = pos % page_size
        if layout == "NHD":
            key_pages[page, slot] = k_rot[b, :, 0, :]
            value_pages[page, slot] = v_raw[b, :, 0, :]
        else:
            key_pages[page, :, slot] = k_rot[b, :, 0, :]
            value_pages[page, :, slot] = v_raw[b, :, 0, :]
    return q_rot


def o_proj(attn_output: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Output projection of a decode step in float32 on the CPU: ``F.linear`` on ``[batch, 1, hidden]``.

    The reference's kernel for this step is Triton-only (kernels/qwen_o_proj_triton.py:25-145) and
    its own test checks it against ``F.linear`` (tests/test_qwen_o_proj_triton.py:19-30); this is
    that checker, evaluated in float32 on the exact input values.
    """

    x = attn_output.detach().to("cpu", torch.float32)
    w = weight.detach().to("cpu", torch.float32)
    b = None if bias is None else bias.detach().to("cpu", torch.float32)
    return torch.nn.functional.linear(x, w, b)


def block_scores(q: torch.Tensor, k: torch.Tensor, *, block_size: int, selector: str) -> torch.Tensor:
    """Score of every block of one head's keys against one query, float32 on the CPU.

    ``q`` is ``[D]``, ``k`` is ``[N, D]``.  Restates the reference's run-time selectors
    (seed_selectors.py:174-196 blocked view and ``qk_block_max``, :252-259 ``block_mean_proxy``):
    the cache is cut into blocks of ``block_size`` tokens (the last one may be short); a block's
    score is the largest q.k over its tokens, or q dotted with the mean of its keys.
    """

    q = q.detach().to("cpu", torch.float32)
    k = k.detach().to("cpu", torch.float32)
    n = int(k.shape[0])
    scores = []
    for start in range(0, n, int(block_size)):
        block = k[start:min(n, start + int(block_size))]
        if selector == "qk_block_max":
            scores.append(torch.matmul(block, q).max())
        elif selector == "block_mean_proxy":
            scores.append(torch.dot(block.mean(dim=0), q))
        else:
            raise ValueError(f"selector {selector!r} is not restated here")
    return torch.stack(scores)


def select_blocks(scores: torch.Tensor, *, seq_len: int, block_size: int, sink_blocks: int, recent_blocks: int,
                  middle_seed_blocks: int, block_order: str) -> List[int]:
    """Seed blocks chosen from block scores (ascending list).

    ``scores`` is ``[heads_sharing_the_kv_head, num_blocks]``: a block's score is the maximum
    over those heads (one head: the reference's per-head rule, seed_selectors.py:347-384).  Sink
    and recent blocks are always kept; the ``middle_seed_blocks`` best other blocks join them,
    ordered by (-score, index), non-finite scores never selecting; the policy's fixed middle
    blocks fill up if fewer blocks have a score.
    """

    num_blocks = math.ceil(int(seq_len) / int(block_size))
    recent_start = num_blocks - int(recent_blocks)
    base = [b for b in range(min(int(sink_blocks), num_blocks))]
    base += [b for b in range(max(recent_start, 0), num_blocks) if b not in base]
    pair = scores.detach().to("cpu", torch.float32).reshape(-1, num_blocks)
    pair = torch.where(torch.isfinite(pair), pair, torch.full_like(pair, -float("inf"))).max(dim=0).values
    ranked = sorted(range(num_blocks), key=lambda b: (-float(pair[b]), b))
    middle: List[int] = []
    for b in ranked:
        if len(middle) >= int(middle_seed_blocks):
            break
        if b in base or not math.isfinite(float(pair[b])):
            continue
        middle.append(b)
    for i in range(int(middle_seed_blocks)):
        if len(middle) >= int(middle_seed_blocks):
            break
        b = int(sink_blocks) + i if block_order == "sequential" else recent_start - 1 - i
        if 0 <= b < num_blocks and b not in base and b not in middle:
            middle.append(b)
    return sorted(base + middle)
