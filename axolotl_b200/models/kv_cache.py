"""KV cache and batched incremental decoding.

Prefill runs the prompts of all sequences as ONE packed varlen row through the training kernels
(each prompt a document), storing the rotated k / v rows of every layer in the cache; every
further token costs one pass with M = batch rows through the GEMMs and the single-query attention
kernel (``ops.functional.decode_attention``) over the live part of the cache. The reference decodes
through Hugging Face ``generate`` (src/axolotl/cli/inference.py, utils/callbacks) with its own cache.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import functional as Fn


class KVCache:
    def __init__(self, model, batch: int, max_len: int):
        cfg = model.config
        dev, dt = model.embed_tokens.device, model.embed_tokens.dtype
        self.L, self.B, self.max_len = cfg.num_hidden_layers, batch, max_len
        att = model.layers[0].self_attn              # local head counts (a tensor-parallel rank holds a slice)
        self.width = att.Hk * att.D
        self.k = torch.zeros(self.L, batch, max_len, self.width, dtype=dt, device=dev)
        self.v = torch.zeros_like(self.k)
        self.lens = torch.zeros(batch, dtype=torch.int32, device=dev)   # live positions per sequence

    def attend(self, layer, qkv, meta, Hq, Hk, D, scale, window=0):
        kq, vq = qkv[:, Hq * D:(Hq + Hk) * D], qkv[:, (Hq + Hk) * D:]
        if meta.decode:
            # one new token per active sequence: row i of qkv belongs to sequence meta.seq[i]
            self.k[layer, meta.seq, meta.pos] = kq
            self.v[layer, meta.seq, meta.pos] = vq
            if meta.all_rows:
                return Fn.decode_attention(qkv, self.k[layer], self.v[layer], meta.lens_after, Hq, Hk, D, scale, window)
            return Fn.decode_attention(qkv, self.k[layer, meta.seq], self.v[layer, meta.seq], meta.lens_after,
                                       Hq, Hk, D, scale, window)
        self.k[layer, meta.seq, meta.pos] = kq         # prefill: packed prompt rows -> (sequence, position)
        self.v[layer, meta.seq, meta.pos] = vq
        return Fn.flash_varlen(qkv, meta.attn.windowed(window) if window else meta.attn, Hq, Hk, D, scale)


class _PrefillMeta:
    decode = False

    def __init__(self, cache, attn, seq, pos):
        self.kv_cache, self.attn, self.seq, self.pos = cache, attn, seq, pos
        self.causal = True


class _DecodeMeta:
    decode = True

    def __init__(self, cache, seq, pos, all_rows):
        self.kv_cache, self.seq, self.pos, self.all_rows = cache, seq, pos, all_rows
        self.lens_after = (pos + 1).to(torch.int32).contiguous()


def _sample(logits, temperature, top_p, top_k, generator):
    if not temperature or temperature <= 0:
        return logits.argmax(-1)
    logits = logits.float() / temperature
    if top_k and top_k > 0:
        kth = logits.topk(min(top_k, logits.shape[-1]), -1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = torch.softmax(logits, -1)
    if top_p is not None and top_p < 1.0:
        sp, si = probs.sort(-1, descending=True)
        keep = sp.cumsum(-1) - sp < top_p
        sp = sp * keep
        probs = torch.zeros_like(probs).scatter_(1, si, sp / sp.sum(-1, keepdim=True))
    return torch.multinomial(probs, 1, generator=generator).squeeze(1)


@torch.no_grad()
def generate_cached(model, prompts, max_new_tokens, temperature=0.0, top_p=1.0, top_k=0, eos_token_id=None,
                    generator=None):
    """Batched decoding with a KV cache. ``prompts``: list of token-id lists (different lengths are
    fine: they are packed, not padded). Returns a list of completion token-id lists (the EOS token,
    when produced, is included and ends its sequence)."""
    dev = model.embed_tokens.device
    n_real = len(prompts)
    if n_real == 0:
        return []
    if min(len(p) for p in prompts) < 1:
        raise ValueError("every prompt needs at least one token")
    prompts = [list(p) for p in prompts]
    if dev.type == "cuda":   # decode steps run the GEMMs with M = batch: keep it a multiple of 8 rows
        prompts += [[int(prompts[0][0])] for _ in range((-n_real) % 8)]
    B = len(prompts)
    lens0 = [len(p) for p in prompts]
    cache = KVCache(model, B, max(lens0) + max_new_tokens)
    was_training = model.training
    model.eval()
    # ---- prefill: all prompts as one packed row
    cu = np.concatenate([[0], np.cumsum(lens0)]).astype(np.int32)
    total = int(cu[-1])
    pad = (-total) % 8                                   # keeps packed rows at the kernels' granularity
    flat = [t for p in prompts for t in p] + [0] * pad
    pos = [i for n in lens0 for i in range(n)] + list(range(pad))
    seq = [b for b, n in enumerate(lens0) for _ in range(n)]
    ids = torch.tensor(flat, dtype=torch.long, device=dev)[None]
    pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)[None]
    attn = Fn.AttnMeta(list(cu) + ([total + pad] if pad else []), dev)
    seq_t = torch.tensor(seq + [0] * pad, dtype=torch.long, device=dev)
    pos_w = torch.tensor(pos[:total] + [cache.max_len - 1] * pad, dtype=torch.long, device=dev)   # pad rows land in a dead slot
    meta = _PrefillMeta(cache, attn, seq_t, pos_w)
    out = model(ids, pos_t, attn_meta=meta, return_logits=False)
    last = torch.tensor([int(c) - 1 for c in cu[1:]], dtype=torch.long, device=dev)
    h_last = out.hidden_states.reshape(-1, out.hidden_states.shape[-1])[last]
    logits = Fn_linear(h_last, model.output_weight())
    cur_len = torch.tensor(lens0, dtype=torch.long, device=dev)
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    done[n_real:] = True                                 # padding sequences never count
    outs = [[] for _ in range(B)]
    all_seq = torch.arange(B, device=dev)
    for step in range(max_new_tokens):
        nxt = _sample(logits, temperature, top_p, top_k, generator)
        nxt_host = nxt.tolist()
        done_host = done.tolist()
        for b in range(n_real):
            if not done_host[b]:
                outs[b].append(int(nxt_host[b]))
        if eos_token_id is not None:
            done = done | (nxt == eos_token_id)
        if bool(done.all()) or step == max_new_tokens - 1:
            break
        # finished sequences keep stepping on their last slot (their outputs are ignored): the batch
        # shape stays fixed, so no re-indexing of the cache is needed
        write_pos = torch.where(done, cur_len - 1, cur_len).clamp(max=cache.max_len - 1)
        dmeta = _DecodeMeta(cache, all_seq, write_pos, True)
        out = model(nxt[None], write_pos.to(torch.int32)[None], attn_meta=dmeta, return_logits=False)
        logits = Fn_linear(out.hidden_states.reshape(B, -1), model.output_weight())
        cur_len = torch.where(done, cur_len, cur_len + 1)
    model.train(was_training)
    return outs[:n_real]


def Fn_linear(h, W):
    from ..ops.lora import linear

    return linear(h, W).float()
