"""Plain torch versions of every function of ``locus_b200.kernels``, same signatures.

Two uses.  (1) ``install()`` swaps them in so that the engine's host logic -- paging,
portions, mixed batches, scheduling, graphs of parts -- runs on the CPU in the ``not gpu``
tests.  (2) The ``gpu`` tests call them on copies of a kernel's inputs as that kernel's
plain reference.  They compute in float32 (or float64 when ``PRECISE`` is set), with plain
loops; they are not a product path and nothing in ``locus_b200`` imports them.
"""
from __future__ import annotations


import torch

import locus_b200.kernels as K

PRECISE = False


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float64 if PRECISE else torch.float32)


def embed_rows(tokens, table, out):
    out.copy_(table[tokens.long()].to(out.dtype))


def attn_chunk_tc_takes(q, head_dim, page_tokens, n_tokens, max_ctx=0):
    return False


def rmsnorm_adds(x):
    return x.dtype == torch.float32 and x.shape[-1] % 4 == 0


def rmsnorm(x, w, eps, out, rows=None, add=None):
    if add is not None and rows is None:
        moe_combine(x[: out.shape[0]], add[0], add[1], add[2])
    elif add is not None:
        x = x.clone()
        moe_combine(x, add[0], add[1], add[2])
    xs = _f(x if rows is None else x[rows.long()])[: out.shape[0]]
    ss = (xs * xs).sum(-1, keepdim=True)
    out.copy_((xs * (1.0 / torch.sqrt(ss / xs.shape[-1] + eps)) * _f(w)).to(out.dtype))


class ExpertLayout(K.ExpertLayout):
    pass


def linear(x, w, out, *, w2=None, bias=None, accumulate=False, row_scale=None, scale_rows=None, x_rows=None, lists_ready=False,
           second_tiles=False,
           x_row_div=1, layout=None, n_rows=None):
    M = out.shape[0] if n_rows is None else n_rows
    if M == 0:
        return
    if x_rows is not None:
        xin = _f(x)[(x_rows[:M].long() // x_row_div)]
    else:
        xin = _f(x)[:M]
    if layout is None:
        y = xin @ _f(w).T
        if w2 is not None:
            u = xin @ _f(w2).T
            y = y / (1.0 + torch.exp(-y)) * u
    else:
        y = torch.zeros(M, w.shape[1], dtype=xin.dtype)
        off = layout.offsets.tolist()
        for e in range(layout.n_experts):
            a, b = off[e], off[e + 1]
            if b > a:
                ye = xin[a:b] @ _f(w[e]).T
                if w2 is not None:
                    ye = ye / (1.0 + torch.exp(-ye)) * (xin[a:b] @ _f(w2[e]).T)
                y[a:b] = ye
    if bias is not None:
        y = y + _f(bias)
    if row_scale is not None:
        rs = row_scale[scale_rows[:M].long()] if scale_rows is not None else row_scale[:M]
        y = y * _f(rs)[:, None]
    if accumulate:
        out[:M] += y.to(out.dtype)
    else:
        out[:M] = y.to(out.dtype)


def rope_kv_write(qkv, positions, inv_freq, q_out, pool, slots, *, n_heads, n_kv_heads, head_dim, rot_dim,
                  interleaved, page_tokens, write_kv=True):
    T = qkv.shape[0]
    x = _f(qkv).view(T, n_heads + 2 * n_kv_heads, head_dim).clone()
    if inv_freq is not None:
        ang = positions[:T].to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
        c, s = _f(torch.cos(ang))[:, None, :], _f(torch.sin(ang))[:, None, :]
        rot = x[:, : n_heads + n_kv_heads, :rot_dim]
        if interleaved:
            x0, x1 = rot[..., 0::2].clone(), rot[..., 1::2].clone()
            rot[..., 0::2] = x0 * c - x1 * s
            rot[..., 1::2] = x0 * s + x1 * c
        else:
            h = rot_dim // 2
            x0, x1 = rot[..., :h].clone(), rot[..., h:].clone()
            rot[..., :h] = x0 * c - x1 * s
            rot[..., h:] = x0 * s + x1 * c
    q_out[:T] = x[:, :n_heads].reshape(T, -1).to(q_out.dtype)
    if not write_kv:
        return
    for t in range(T):
        page, off = int(slots[t]) // page_tokens, int(slots[t]) % page_tokens
        pool[page, 0, :, off, :] = x[t, n_heads : n_heads + n_kv_heads].to(pool.dtype)
        pool[page, 1, :, off, :] = x[t, n_heads + n_kv_heads :].to(pool.dtype)


def _attend_one(q, pool, table, p, kvh, page_tokens, window, scale):
    lo = max(0, p - window + 1) if window > 0 else 0
    ts = list(range(lo, p + 1))
    pages = [int(table[t // page_tokens]) for t in ts]
    assert all(pg >= 0 for pg in pages), "attention reads a page that was given back"
    k = torch.stack([_f(pool[pg, 0, kvh, t % page_tokens]) for pg, t in zip(pages, ts)])
    v = torch.stack([_f(pool[pg, 1, kvh, t % page_tokens]) for pg, t in zip(pages, ts)])
    s = (k @ _f(q)) * scale
    a = torch.softmax(s, dim=0)
    return a @ v


def _attn(q, pool, out, seg_list, *, seg_q0, seg_qn, seg_ctx, block_table, n_heads, n_kv_heads, head_dim,
          page_tokens, window, scale):
    group = n_heads // n_kv_heads
    for seg in seg_list:
        q0, qn, ctx = int(seg_q0[seg]), int(seg_qn[seg]), int(seg_ctx[seg])
        for i in range(qn):
            for h in range(n_heads):
                qv = q[q0 + i].view(n_heads, head_dim)[h]
                o = _attend_one(qv, pool, block_table[seg], ctx + i, h // group, page_tokens, window, scale)
                out[q0 + i].view(n_heads, head_dim)[h] = o.to(out.dtype)


def attn_chunk(q, pool, out, *, seg_q0, seg_qn, seg_ctx, block_table, items, n_items, n_heads, n_kv_heads,
               head_dim, page_tokens, window, scale):
    segs = sorted({int(items[i, 0]) for i in range(n_items)})
    _attn(q, pool, out, segs, seg_q0=seg_q0, seg_qn=seg_qn, seg_ctx=seg_ctx, block_table=block_table,
          n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, page_tokens=page_tokens, window=window,
          scale=scale)


def attn_chunk_mma_splits(n_items, n_heads, max_ctx):
    return 1


def attn_chunk_mma(q, pool, out, *, seg_q0, seg_qn, seg_ctx, block_table, items, n_items, n_heads, n_kv_heads,
                   head_dim, page_tokens, window, scale, n_splits=1, part_o=None, part_ml=None):
    attn_chunk(q, pool, out, seg_q0=seg_q0, seg_qn=seg_qn, seg_ctx=seg_ctx, block_table=block_table, items=items,
               n_items=n_items, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, page_tokens=page_tokens,
               window=window, scale=scale)


def attn_decode(q, pool, out, *, seg_q0, seg_qn, seg_ctx, block_table, items, n_items, n_heads, n_kv_heads,
                head_dim, page_tokens, window, scale, part_o, part_ml, counters, max_splits):
    segs = [int(items[i]) for i in range(n_items)]
    for s in segs:
        assert int(seg_ctx[s]) // K.DECODE_SPLIT + 1 <= max_splits
    _attn(q, pool, out, segs, seg_q0=seg_q0, seg_qn=seg_qn, seg_ctx=seg_ctx, block_table=block_table,
          n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, page_tokens=page_tokens, window=window,
          scale=scale)


def _select(logits_row, top_k, renorm, scale, score_fn, sel_bias, n_group, n_group_used):
    """The selection rule of csrc/moe_route.cu (select_token) for one token."""
    E = logits_row.shape[0]
    r = logits_row
    if score_fn == "softmax":
        e = torch.exp(r - r.max())
        p = e / e.sum()
    else:
        p = 1.0 / (1.0 + torch.exp(-r))
    sel = p.clone() if sel_bias is None else p + sel_bias.to(p.dtype).cpu()
    sel = torch.where(torch.isnan(sel), torch.full_like(sel, -3.0e38), sel)
    if n_group > 1:
        per = E // n_group
        gs = []
        for g in range(n_group):
            top2 = torch.sort(torch.cat([sel[g * per : (g + 1) * per], torch.full((2,), -1e30, dtype=sel.dtype)]), descending=True).values
            gs.append(float(top2[0]) + (float(top2[1]) if per > 1 else 0.0))
        keep = []
        for _ in range(n_group_used):
            keep.append(max((g for g in range(n_group) if g not in keep), key=lambda g: (gs[g], -g)))
        for x in range(E):
            if x // per not in keep:
                sel[x] = -1e30
    picked = []
    for _ in range(top_k):
        best = max((x for x in range(E) if x not in picked), key=lambda x: (float(sel[x]), -x))
        picked.append(best)
    wsum = sum(p[x] for x in picked) if renorm else 1.0
    return picked, [float(p[x] / wsum * scale) for x in picked]


def router_topk(h, w_router, w_gate, ids, wts, gamma, *, top_k, renorm, scale=1.0, scratch=None, score_fn="softmax",
                sel_bias=None, n_group=1, n_group_used=1):
    T = h.shape[0]
    r = _f(h) @ _f(w_router).T
    for t in range(T):
        picked, w = _select(r[t], top_k, renorm, scale, score_fn, sel_bias, n_group, n_group_used)
        for j, e in enumerate(picked):
            ids[t * top_k + j] = e
            wts[t * top_k + j] = w[j]
    if w_gate is not None:
        z = _f(h) @ _f(w_gate).reshape(-1)
        gamma[:T] = (1.0 / (1.0 + torch.exp(-z))).to(gamma.dtype)


def router_logits(h, w_all, logits):
    T, n = h.shape[0], w_all.shape[0]
    logits[:T, :n] = (_f(h) @ _f(w_all).T).to(logits.dtype)


def router_select(logits, n_experts, has_gate, ids, wts, gamma, *, n_tokens, top_k, renorm, scale=1.0,
                  score_fn="softmax", sel_bias=None, n_group=1, n_group_used=1):
    lg = _f(logits[:n_tokens, :n_experts])
    for t in range(n_tokens):
        picked, w = _select(lg[t], top_k, renorm, scale, score_fn, sel_bias, n_group, n_group_used)
        for j, e in enumerate(picked):
            ids[t * top_k + j] = e
            wts[t * top_k + j] = w[j]
    if has_gate:
        z = _f(logits[:n_tokens, n_experts])
        gamma[:n_tokens] = (1.0 / (1.0 + torch.exp(-z))).to(gamma.dtype)


def route_small_takes(n_tokens, top_k, n_experts):
    return n_tokens <= 16 and n_tokens * top_k <= 1024 and n_experts <= 512


def route_small(logits, n_experts, has_gate, ids, wts, gamma, layout, *, n_tokens, top_k, renorm, scale=1.0,
                tile_m=None, **rule):
    router_select(logits, n_experts, has_gate, ids, wts, gamma, n_tokens=n_tokens, top_k=top_k, renorm=renorm,
                  scale=scale, **rule)
    moe_sort(ids, n_tokens * top_k, layout, tile_m)


def route_fused_small(h, w_all, logits, n_experts, has_gate, ids, wts, gamma, layout, counter, *, n_tokens, tile_m=None,
                      **rule):
    router_logits(h[:n_tokens], w_all, logits)
    route_small(logits, n_experts, has_gate, ids, wts, gamma, layout, n_tokens=n_tokens, tile_m=tile_m, **rule)


def moe_sort(ids, n_pairs, layout, tile_m=None, tile2_m=0):
    if tile_m is not None:
        layout.tile_m = tile_m
    layout.tile2_m = tile2_m
    E, tm = layout.n_experts, layout.tile_m
    idl = ids[:n_pairs].tolist()
    pos = 0
    tile = tile2 = 0
    for e in range(E):
        mine = [p for p, x in enumerate(idl) if x == e]
        layout.counts[e] = len(mine)
        layout.offsets[e] = pos
        for i in range(0, len(mine), tm):
            layout.tile_expert[tile] = e
            layout.tile_row0[tile] = pos + i
            layout.tile_rows[tile] = min(tm, len(mine) - i)
            tile += 1
        for i in range(0, len(mine), tile2_m) if tile2_m else ():
            layout.tile2_expert[tile2] = e
            layout.tile2_row0[tile2] = pos + i
            layout.tile2_rows[tile2] = min(tile2_m, len(mine) - i)
            tile2 += 1
        for p in mine:
            layout.sorted_pair[pos] = p
            layout.pair_pos[p] = pos
            pos += 1
    layout.offsets[E] = pos
    layout.n_tiles[0] = tile
    if tile2_m:
        layout.n_tiles2[0] = tile2


def moe_combine(x, pair_out, pair_pos, top_k):
    T = x.shape[0]
    for t in range(T):
        acc = torch.zeros_like(x[t])
        for s in range(top_k):
            acc = acc + pair_out[int(pair_pos[t * top_k + s])].to(acc.dtype)
        x[t] += acc


def gather_rows(src, idx, div, out, n):
    out[:n] = src[(idx[:n].long() // div)]


def apply_penalties(logits, history, repeat, freq, presence):
    R, V = logits.shape
    for r in range(R):
        rp, fp, pp = float(repeat[r]), float(freq[r]), float(presence[r])
        if rp == 1.0 and fp == 0.0 and pp == 0.0:
            continue
        counts = {}
        for t in history[r].tolist():
            if 0 <= t < V:
                counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            l = float(logits[r, t])
            if rp != 1.0:
                l = l / rp if l > 0 else l * rp
            logits[r, t] = l - (fp * c + pp)


def sample(logits, *, temperature, top_k, top_p, min_p, seeds, counters, out, kept_count=None):
    """Greedy rows exactly; stochastic rows by torch's generator seeded from (seed, counter)
    over the same kept set (the device kernel has its own counter-based generator)."""
    R, V = logits.shape
    for r in range(R):
        row = logits[r].double()
        T = float(temperature[r])
        if not T > 0:
            out[r] = int(torch.argmax(row))  # first maximum
            continue
        keep = torch.ones(V, dtype=torch.bool)
        k = int(top_k[r])
        if 0 < k < V:
            thr = torch.sort(row, descending=True).values[k - 1]
            keep &= row >= thr
        w = torch.where(keep, torch.exp((row - row.max()) / T), torch.zeros_like(row))
        tp = float(top_p[r])
        if tp < 1.0:
            sw, _ = torch.sort(w, descending=True)
            cum = torch.cumsum(sw, 0)
            j = int(torch.nonzero(cum >= tp * w.sum())[0])
            keep &= w >= sw[j]
        mp = float(min_p[r])
        if mp > 0:
            keep &= w >= mp * w.max()
        w = torch.where(keep, w, torch.zeros_like(w))
        g = torch.Generator().manual_seed((int(seeds[r]) * 1000003 + int(counters[r])) & 0x7FFFFFFF)
        out[r] = int(torch.multinomial(w / w.sum(), 1, generator=g))
        if kept_count is not None:
            kept_count[r] = int(keep.sum())


_NAMES = ["embed_rows", "rmsnorm", "rmsnorm_adds", "attn_chunk_tc_takes", "linear", "rope_kv_write", "attn_chunk", "attn_chunk_mma", "attn_decode", "router_topk", "router_logits", "router_select",
          "moe_sort", "route_small", "route_small_takes", "route_fused_small", "moe_combine", "gather_rows", "apply_penalties", "sample"]


def install(monkeypatch) -> None:
    """Replace the CUDA entry points by the functions of this file (pytest monkeypatch)."""
    g = globals()
    for n in _NAMES:
        monkeypatch.setattr(K, n, g[n])
    from locus_b200.csrc import build
    monkeypatch.setattr(build, "ensure", lambda names, verbose=True: None)
