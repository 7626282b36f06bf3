"""Plain float32 references of single kernels, written with torch on the CPU, and
helpers that lay test data out the way the kernels read it (pages, block tables)."""

from __future__ import annotations


import torch


def ref_paged_attention(q, k_seq, v_seq, positions, token_req, nq, nkv, d, scale, window=0):
    """q [n, nq*d]; k_seq[r], v_seq[r]: [len_r, nkv, d] per request; the query of token t
    (request token_req[t], position positions[t]) sees keys lo..position of its request."""
    n = q.shape[0]
    out = torch.zeros(n, nq * d, dtype=torch.float64)
    q = q.double().reshape(n, nq, d)
    group = nq // nkv
    for t in range(n):
        r, pos = int(token_req[t]), int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        k = k_seq[r][lo:pos + 1].double()
        v = v_seq[r][lo:pos + 1].double()
        for h in range(nq):
            hk = h // group
            s = (k[:, hk, :] @ q[t, h]) * scale
            w = torch.softmax(s, dim=0)
            out[t, h * d:(h + 1) * d] = (w[:, None] * v[:, hk, :]).sum(0)
    return out


def build_pages(k_seq, v_seq, page_size, num_pages, nkv, d, dtype, device, seed=0):
    """Scatters per-request key/value sequences into pages taken in a shuffled order;
    unused pages hold large values, so that reading a wrong page shows."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(num_pages, generator=g).tolist()
    k_pages = torch.full((num_pages, nkv, page_size, d), 50.0, dtype=torch.float32)
    v_pages = torch.full((num_pages, nkv, page_size, d), -50.0, dtype=torch.float32)
    max_blocks = max(-(-k.shape[0] // page_size) for k in k_seq) + 1
    table = torch.full((len(k_seq), max_blocks), -1, dtype=torch.int32)
    for r, (k, v) in enumerate(zip(k_seq, v_seq)):
        for b in range(-(-k.shape[0] // page_size)):
            page = order.pop()
            table[r, b] = page
            rows = k[b * page_size:(b + 1) * page_size]
            k_pages[page, :, :rows.shape[0], :] = rows.transpose(0, 1)
            v_pages[page, :, :rows.shape[0], :] = v[b * page_size:(b + 1) * page_size].transpose(0, 1)
    return (k_pages.to(dtype).to(device).contiguous(), v_pages.to(dtype).to(device).contiguous(),
            table.to(device))
