"""Inputs for the attention kernels built directly with torch, and their plain float64 answer."""
import math

import torch

PAGE = 64


def attention_case(seq_lens_new, pos0, nh, nkvh, dh, dtype, tile_tokens, seed=0, device="cuda", scale_key=None):
    """A ragged batch: sequence b has pos0[b] tokens in the cache and seq_lens_new[b] new ones.
    Pages are handed out in a scrambled order so that a wrong page lookup shows.
    scale_key = (b, position, factor) multiplies one key (and the matching query direction) so that
    one far score stands out."""
    g = torch.Generator().manual_seed(seed)
    B = len(seq_lens_new)
    total = [p + n for p, n in zip(pos0, seq_lens_new)]
    n_pages_seq = [(t + PAGE - 1) // PAGE for t in total]
    n_pages = sum(n_pages_seq) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max(n_pages_seq) + 1
    table = torch.zeros((B, max_pages), dtype=torch.int32)
    k_seq = [torch.randn(total[b], nkvh, dh, generator=g) for b in range(B)]
    v_seq = [torch.randn(total[b], nkvh, dh, generator=g) for b in range(B)]
    nt = sum(seq_lens_new)
    q = torch.randn(nt, nh, dh, generator=g)
    if scale_key is not None:
        b, p, f = scale_key
        k_seq[b][p] *= f
    kc = torch.randn(n_pages, nkvh, PAGE, dh, generator=g)      # garbage where nothing was written
    vc = torch.randn(n_pages, nkvh, PAGE, dh, generator=g)
    nxt = 0
    for b in range(B):
        for i in range(n_pages_seq[b]):
            pg = perm[nxt]
            nxt += 1
            table[b, i] = pg
            lo, hi = i * PAGE, min(total[b], (i + 1) * PAGE)
            kc[pg, :, : hi - lo] = k_seq[b][lo:hi].transpose(0, 1)
            vc[pg, :, : hi - lo] = v_seq[b][lo:hi].transpose(0, 1)
    tok_pos, tile_seq, tile_t0, tile_nq = [], [], [], []
    t = 0
    for b in range(B):
        tok_pos += list(range(pos0[b], total[b]))
        for off in range(0, seq_lens_new[b], tile_tokens):
            tile_seq.append(b)
            tile_t0.append(t + off)
            tile_nq.append(min(tile_tokens, seq_lens_new[b] - off))
        t += seq_lens_new[b]
    to = lambda x, dt: x.to(dt).to(device)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    case = dict(q=to(q, dtype).contiguous(), kc=to(kc, dtype), vc=to(vc, dtype), table=table.to(device),
                tok_pos=i32(tok_pos), tile_seq=i32(tile_seq), tile_t0=i32(tile_t0), tile_nq=i32(tile_nq),
                tiles=len(tile_seq), nt=nt, max_pages=max_pages, nh=nh, nkvh=nkvh, dh=dh)
    # the plain answer from the values as stored (rounded to dtype)
    ref = torch.zeros(nt, nh, dh, dtype=torch.float64)
    qd = q.to(dtype).double()
    group = nh // nkvh
    t = 0
    for b in range(B):
        kd, vd = k_seq[b].to(dtype).double(), v_seq[b].to(dtype).double()
        for i in range(seq_lens_new[b]):
            p = pos0[b] + i
            for h in range(nh):
                s = (kd[: p + 1, h // group] @ qd[t, h]) / math.sqrt(dh)
                ref[t, h] = torch.softmax(s, 0) @ vd[: p + 1, h // group]
            t += 1
    case["ref"] = ref
    return case
