"""Sampling-side device ops: greedy argmax, top-k/top-p sampling, MTP verification, multi-step
input advance, Omni-Attention ring-window slots (``csrc/kernels/sampler_misc.cu``)."""
from __future__ import annotations

import torch

from . import _native as nat


def argmax(logits, vocab_offset=0, want_max=False):
    """Greedy token per row.  ``want_max`` also returns the max logit (vocab-parallel heads exchange
    (max, index) pairs instead of full logits)."""
    if not logits.is_cuda:
        mx, idx = logits.float().max(dim=-1)
        idx = idx + vocab_offset
        return (idx, mx) if want_max else idx
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    mx = torch.empty(B, dtype=torch.float32, device=logits.device) if want_max else None
    rc = nat.lib().omni_argmax(nat.ptr(logits), nat.c_int(1 if logits.dtype == torch.bfloat16 else 0), nat.c_int(B),
                               nat.c_int(V), nat.c_int(logits.stride(0)), nat.c_int(vocab_offset), nat.ptr(ids),
                               nat.ptr(mx), nat.stream())
    nat.check_rc(rc, "omni_argmax")
    return (ids, mx) if want_max else ids


def apply_penalties_ref(logits, hist, prompt_len, rep, freq, pres):
    """fp32 reference of :func:`apply_penalties` (returns a new tensor)."""
    B, V = logits.shape
    out = logits.float().clone()
    for b in range(B):
        r, f, p = float(rep[b]), float(freq[b]), float(pres[b])
        if r == 1.0 and f == 0.0 and p == 0.0:
            continue
        h = hist[b]
        h = h[h >= 0].long()
        npr = int(prompt_len[b])
        seen = torch.zeros(V, dtype=torch.bool, device=logits.device)
        seen[h] = True
        cnt = torch.zeros(V, dtype=torch.float32, device=logits.device)
        cnt.scatter_add_(0, h[npr:], torch.ones(h[npr:].numel(), device=logits.device))
        row = out[b]
        row = torch.where(seen, torch.where(row > 0, row / r, row * r), row)
        row = row - f * cnt - p * (cnt > 0).float()
        out[b] = row
    return out.to(logits.dtype)


_pen_scratch = {}


def apply_penalties(logits, hist, prompt_len, rep, freq, pres):
    """Repetition / frequency / presence penalties (omni/models/common/layers/sampler.py:143-200), in place on CUDA.

    ``hist`` [B, L] int32: each row's prompt tokens followed by its output tokens, -1 padded; ``prompt_len`` [B]
    int32; ``rep`` / ``freq`` / ``pres`` [B] fp32 (1, 0, 0 = no penalty).  Returns the penalised logits."""
    if not logits.is_cuda:
        return apply_penalties_ref(logits, hist, prompt_len, rep, freq, pres)
    B, V = logits.shape
    assert logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    key = logits.device.index
    sc = _pen_scratch.get(key)
    if sc is None or sc.numel() < B * V:
        sc = _pen_scratch[key] = torch.empty(B * V, dtype=torch.int32, device=logits.device)
    hist = hist.contiguous()
    rc = nat.lib().omni_apply_penalties(
        nat.ptr(logits), nat.c_int(1 if logits.dtype == torch.bfloat16 else 0), nat.c_int(B), nat.c_int(V),
        nat.c_int(logits.stride(0)), nat.ptr(hist), nat.c_int(hist.shape[1]), nat.ptr(prompt_len), nat.ptr(rep),
        nat.ptr(freq), nat.ptr(pres), nat.ptr(sc), nat.stream())
    nat.check_rc(rc, "omni_apply_penalties")
    return logits


def sample_topk_topp_ref(logits, temperature, top_k, top_p, uniform):
    """Reference with the same semantics as the kernel: keep {p >= tau}, tau = max(k-th largest p,
    largest threshold whose kept mass >= top_p); inverse CDF in index order."""
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int64)
    for b in range(B):
        t = float(temperature[b]) if temperature is not None else 1.0
        if t < 1e-5:
            out[b] = int(logits[b].float().argmax())
            continue
        p = torch.softmax(logits[b].double() / t, dim=-1)
        keep = torch.ones(V, dtype=torch.bool)
        k = int(top_k[b]) if top_k is not None else 0
        sp, _ = p.sort(descending=True)
        tau = 0.0
        if 0 < k < V:
            tau = max(tau, float(sp[k - 1]))
        pp = float(top_p[b]) if top_p is not None else 1.0
        if pp < 1.0:
            cs = sp.cumsum(0)
            j = int((cs >= pp).nonzero()[0])
            tau = max(tau, float(sp[j]))
        keep = p >= tau * (1 - 1e-6)
        pk = torch.where(keep, p, torch.zeros_like(p))
        cdf = pk.cumsum(0)
        target = float(uniform[b]) * float(cdf[-1])
        idx = int((cdf >= target).nonzero()[0]) if target > 0 else int(keep.nonzero()[0])
        out[b] = idx
    return out


def sample_topk_topp(logits, temperature=None, top_k=None, top_p=None, uniform=None, generator=None):
    """Temperature / top-k / top-p sampling, one uniform random number per row.  Rows with
    temperature ~ 0 are greedy."""
    B, V = logits.shape
    if uniform is None:
        uniform = torch.rand(B, device=logits.device, generator=generator)
    if not logits.is_cuda:
        return sample_topk_topp_ref(logits, temperature, top_k, top_p, uniform)
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    rc = nat.lib().omni_sample_topk_topp(
        nat.ptr(logits), nat.c_int(1 if logits.dtype == torch.bfloat16 else 0), nat.c_int(B), nat.c_int(V),
        nat.c_int(logits.stride(0)), nat.ptr(temperature), nat.ptr(top_k), nat.ptr(top_p), nat.ptr(uniform),
        nat.ptr(ids), nat.stream())
    nat.check_rc(rc, "omni_sample_topk_topp")
    return ids


def mtp_verify_ref(input_ids, forward_tokens, accept_uniform=None, control_accept_rate=-1.0):
    B, n = input_ids.shape
    if accept_uniform is not None:
        accepted = accept_uniform.view(B, n - 1) < control_accept_rate
    else:
        accepted = input_ids[:, 1:] == forward_tokens[:, :-1]
    mask = torch.cat([accepted.int(), torch.zeros(B, 1, dtype=torch.int32, device=input_ids.device)], dim=1)
    accepted_num = mask.argmin(dim=1).int()
    offs = torch.arange(n, device=input_ids.device)
    out = torch.where(offs[None, :] <= accepted_num[:, None], forward_tokens, torch.full_like(forward_tokens, -1))
    last = (torch.arange(B, device=input_ids.device) * n + accepted_num).int()
    return out, accepted_num, last, forward_tokens.clone()


def mtp_verify(input_ids, forward_tokens, accept_uniform=None, control_accept_rate=-1.0):
    """MTP draft verification (omni/models/common/layers/sampler.py:812-840): input_ids [B, 1+k] =
    last accepted token followed by k drafts, forward_tokens [B, 1+k] = the main model's token at every
    position.  Draft i is accepted iff it equals the model's token at position i-1.  Returns
    (output tokens with -1 after the first rejection, accepted_num, last_accepted_index, drafter inputs)."""
    if not input_ids.is_cuda:
        return mtp_verify_ref(input_ids, forward_tokens, accept_uniform, control_accept_rate)
    B, n = input_ids.shape
    dev = input_ids.device
    out = torch.empty(B, n, dtype=torch.int64, device=dev)
    acc = torch.empty(B, dtype=torch.int32, device=dev)
    last = torch.empty(B, dtype=torch.int32, device=dev)
    nxt = torch.empty(B, n, dtype=torch.int64, device=dev)
    rc = nat.lib().omni_mtp_verify(nat.ptr(input_ids.contiguous()), nat.ptr(forward_tokens.contiguous()), nat.c_int(B),
                                   nat.c_int(n), nat.ptr(out), nat.ptr(acc), nat.ptr(last), nat.ptr(nxt),
                                   nat.ptr(accept_uniform), nat.c_float(control_accept_rate), nat.stream())
    nat.check_rc(rc, "omni_mtp_verify")
    return out, acc, last, nxt


def step_advance(positions, seq_lens, slots, block_table, block_size, tokens_per_req=1, advance=None):
    """In place: every live row (seq_len > 0) grows by ``advance[b]`` (default 1) tokens; positions and
    cache slots of its next ``tokens_per_req`` inputs are recomputed from the block table."""
    B = seq_lens.shape[0]
    if not seq_lens.is_cuda:
        for b in range(B):
            if int(seq_lens[b]) <= 0:
                continue
            adv = int(advance[b]) if advance is not None else 1
            seq_lens[b] += adv
            for j in range(tokens_per_req):
                pos = int(seq_lens[b]) - tokens_per_req + j
                positions[b * tokens_per_req + j] = pos
                slots[b * tokens_per_req + j] = int(block_table[b, pos // block_size]) * block_size + pos % block_size
        return
    rc = nat.lib().omni_step_advance(nat.ptr(positions), nat.ptr(seq_lens), nat.ptr(slots), nat.ptr(block_table),
                                     nat.c_int(block_table.stride(0)), nat.c_int(block_size), nat.c_int(B),
                                     nat.c_int(tokens_per_req), nat.ptr(advance), nat.stream())
    nat.check_rc(rc, "omni_step_advance")


def omni_attn_slots_ref(seq_lens, prompt_lens, block_table, block_size, sink, recent):
    B = seq_lens.shape[0]
    slots = torch.full((B,), -1, dtype=torch.int64)
    eff = torch.zeros(B, dtype=torch.int32)
    st, rt = sink * block_size, recent * block_size
    cap = st + rt
    for b in range(B):
        L = int(seq_lens[b])
        if L <= 0:
            continue
        if L <= cap:
            pos = L - 1
        else:
            base = max(cap, int(prompt_lens[b])) + 1
            pos = (L - base) % rt + st
        slots[b] = int(block_table[b, pos // block_size]) * block_size + pos % block_size
        eff[b] = min(L, cap)
    return slots, eff


def omni_attn_slots(seq_lens, prompt_lens, block_table, block_size, sink, recent):
    """Slot of the newest token in a compressed (sink + recent window) layer, and the number of tokens
    that layer attends over (omni/accelerators/cache/utils.py:36-50)."""
    if not seq_lens.is_cuda:
        return omni_attn_slots_ref(seq_lens, prompt_lens, block_table, block_size, sink, recent)
    B = seq_lens.shape[0]
    slots = torch.empty(B, dtype=torch.int64, device=seq_lens.device)
    eff = torch.empty(B, dtype=torch.int32, device=seq_lens.device)
    rc = nat.lib().omni_omni_attn_slots(nat.ptr(seq_lens), nat.ptr(prompt_lens), nat.ptr(block_table),
                                        nat.c_int(block_table.stride(0)), nat.c_int(block_size), nat.c_int(sink),
                                        nat.c_int(recent), nat.c_int(B), nat.ptr(slots), nat.ptr(eff), nat.stream())
    nat.check_rc(rc, "omni_omni_attn_slots")
    return slots, eff
