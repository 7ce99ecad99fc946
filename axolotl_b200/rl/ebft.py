"""Energy-based fine-tuning (EBFT), structured mode: GRPO whose reward is the match between the
FEATURES of a sampled completion and those of the ground-truth completion under a frozen copy
of the policy ("Matching Features, Not Tokens", Jelassi et al. 2026; reference:
src/axolotl/core/trainers/ebft/trainer.py:43-420 and rewards.py:14-264).

    reward_i = alignment_coef * 2 cos(phi(gen_i), phi(gt)) - diversity_coef * 2 mean_{j != i} <phi(gen_i), phi(gen_j)>

``phi`` concatenates the residual stream at a few depths (``feature_layers`` as fractions of the
layer count), pooled per sequence (``last_token`` / ``mean_pooling`` / ``completion_mean`` /
``concat`` of the quartile positions), optionally whitened per prompt group with the SVD of the
generated embeddings. The frozen feature network is the policy itself with its adapters
switched off (or a frozen copy for a full fine-tune). All sequences of a batch are scored in
packed varlen rows: one forward per ~``tokens_per_row`` tokens instead of one per padded batch.
Strided mode (unstructured text) is expressed through the same machinery: every ``stride`` tokens of
a document is an anchor; the ``context_length`` tokens before it are the prompt and the
``generate_max_len`` tokens after it the ground truth (``strided_records``), sampled
``n_samples_per_prompt`` times with the leave-one-out (RLOO) baseline. The reference evaluates all
anchors of a document in one forward pass with a block-structured mask
(src/axolotl/core/trainers/ebft/strided.py); here each anchor is its own short packed document.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..models.layers import disable_adapters
from ..ops import functional as Fn


def pool_features(h, method, prompt_len):
    """h: [len, D] hidden states of one sequence -> [D] (or [3D] for ``concat``)."""
    n = h.shape[0]
    if method == "last_token":
        return h[-1]
    if method == "mean_pooling":
        return h.float().mean(0).to(h.dtype)
    if method == "completion_mean":
        comp = h[min(prompt_len, n - 1):]
        return comp.float().mean(0).to(h.dtype)
    if method == "concat":
        q = [min(max(n * k // 4, 0), n - 1) for k in (1, 2, 3)]
        return torch.cat([h[q[0]], h[q[1]], h[q[2]]], -1)
    raise ValueError(f"Unknown embed_method: {method}")


def whiten(phi, phi_gt, tol=1e-5):
    """Whitening transform estimated from the generated embeddings [n, D] (pseudo-inverse of their
    singular values), applied to them and to the ground-truth embedding [1, D]."""
    pf, gf = phi.float(), phi_gt.float()
    try:
        U, S, _ = torch.linalg.svd(pf.T, full_matrices=False)
    except Exception:
        return F.normalize(pf, dim=-1), F.normalize(gf, dim=-1)
    inv = torch.where(S > tol * S.max(), 1.0 / (S + 1e-12), torch.zeros_like(S))
    W = (U * inv[None]) @ U.T
    return pf @ W, gf @ W


def feature_rewards(gen_emb, gt_emb, n, alignment_coef=1.0, diversity_coef=1.0, use_whitening=False):
    """gen_emb [P*n, D], gt_emb [P, D] -> (rewards [P*n], metrics)."""
    P = gt_emb.shape[0]
    if use_whitening and n > 1:
        g_l, t_l = [], []
        for i in range(P):
            a, b = whiten(gen_emb[i * n:(i + 1) * n], gt_emb[i:i + 1])
            g_l.append(a)
            t_l.append(b)
        gen, gt = torch.cat(g_l), torch.cat(t_l)
    else:
        gen, gt = F.normalize(gen_emb.float(), dim=-1), F.normalize(gt_emb.float(), dim=-1)
    D = gen.shape[-1]
    if gen.is_cuda and (D + 2 * n + 1) * 4 <= 200 * 1024:
        # one kernel for both terms (no [n, n] similarity matrix): csrc/ebft.cu
        from ..ops import _lib

        gen_c, gt_c = gen.contiguous(), gt.contiguous()
        align = torch.empty(P * n, dtype=torch.float32, device=gen.device)
        div = torch.empty_like(align)
        _lib.check_rc(_lib.cuda_lib().axb_ebft_rewards(gen_c.data_ptr(), gt_c.data_ptr(), align.data_ptr(), div.data_ptr(),
                                                       P, n, D, 0, _lib.stream_ptr()), "ebft_rewards")
    elif n > 1:
        align = 2 * F.cosine_similarity(gen, gt.repeat_interleave(n, 0), dim=-1)
        g3 = gen.view(P, n, -1)
        sims = g3 @ g3.transpose(1, 2)
        sims = sims.masked_fill(torch.eye(n, dtype=torch.bool, device=sims.device)[None], 0.0)
        div = 2 * (sims.sum(-1) / (n - 1)).reshape(-1)
    else:
        align = 2 * F.cosine_similarity(gen, gt.repeat_interleave(n, 0), dim=-1)
        div = torch.zeros_like(align)
    cfm = ((gen.view(P, n, -1).mean(1) - gt) ** 2).sum(-1).mean()
    rewards = alignment_coef * align - diversity_coef * div
    return rewards, {"ebft/alignment": float(align.mean()), "ebft/diversity": float(div.mean()),
                     "ebft/cfm_loss": float(cfm), "ebft/reward": float(rewards.mean())}


class FeatureMatchingReward:
    """Reward callable for the rollout producer (same keyword interface as text reward functions;
    uses ``prompt_ids`` / ``completion_ids`` and the dataset's ``ground_truth`` column)."""

    __name__ = "ebft_feature_matching"

    def __init__(self, model, tokenizer, settings: dict, num_generations: int, feature_model=None,
                 tokens_per_row: int = 16384):
        self.model, self.tok, self.n = model, tokenizer, num_generations
        self.feature_model = feature_model      # frozen copy (full fine-tune); None = policy with adapters off
        s = dict(settings or {})
        L = model.config.num_hidden_layers
        self.layers = [int(f * L) for f in (s.get("feature_layers") or [0.25, 0.5, 0.75])]
        self.method = s.get("embed_method") or "last_token"
        self.whiten = bool(s.get("use_whitening"))
        self.a = 1.0 if s.get("alignment_coef") is None else float(s["alignment_coef"])
        self.d = 1.0 if s.get("diversity_coef") is None else float(s["diversity_coef"])
        self.tokens_per_row = tokens_per_row
        self.last_metrics = {}

    def _gt_ids(self, gt):
        if isinstance(gt, str):
            if self.tok is None:
                raise ValueError("string ground_truth needs a tokenizer")
            return list(self.tok(gt, add_special_tokens=False)["input_ids"])
        return [int(t) for t in gt]

    @torch.no_grad()
    def embed(self, seqs, prompt_lens):
        """seqs: list of token-id lists -> [len(seqs), D'] features."""
        net = self.feature_model or self.model
        dev = net.embed_tokens.device
        was = net.training
        net.eval()
        out = [None] * len(seqs)
        i = 0
        from contextlib import nullcontext

        ctx = disable_adapters() if self.feature_model is None else nullcontext()
        with ctx:
            while i < len(seqs):
                j, tot = i, 0
                while j < len(seqs) and (j == i or tot + len(seqs[j]) <= self.tokens_per_row):
                    tot += len(seqs[j])
                    j += 1
                cu = [0]
                for s in seqs[i:j]:
                    cu.append(cu[-1] + len(s))
                pad = (-cu[-1]) % 8     # rows of the packed stream stay 16-byte multiples; padding is its own document
                flat = [t for s in seqs[i:j] for t in s] + [0] * pad
                pos = [p for s in seqs[i:j] for p in range(len(s))] + list(range(pad))
                ids = torch.tensor(flat, dtype=torch.long)[None]
                pos_t = torch.tensor(pos, dtype=torch.int32)[None]
                meta = Fn.AttnMeta(cu + ([cu[-1] + pad] if pad else []), dev)
                res = net(ids, pos_t, attn_meta=meta, return_logits=False, capture_hidden=self.layers)
                feats = torch.cat([res.captured[l].reshape(-1, res.captured[l].shape[-1]) for l in self.layers], -1)
                for k in range(i, j):
                    a, b = cu[k - i], cu[k - i + 1]
                    out[k] = pool_features(feats[a:b], self.method, prompt_lens[k])
                i = j
        net.train(was)
        return torch.stack(out)

    def __call__(self, prompts=None, completions=None, completion_ids=None, ground_truth=None, prompt_ids=None, **kw):
        if ground_truth is None or prompt_ids is None:
            return [0.0] * len(completion_ids)
        n = self.n
        gen = [list(p) + list(c) for p, c in zip(prompt_ids, completion_ids)]
        gen_pl = [len(p) for p in prompt_ids]
        gt = [list(prompt_ids[k]) + self._gt_ids(ground_truth[k]) for k in range(0, len(prompt_ids), n)]
        gt_pl = [len(prompt_ids[k]) for k in range(0, len(prompt_ids), n)]
        emb = self.embed(gen + gt, gen_pl + gt_pl)
        r, m = feature_rewards(emb[: len(gen)], emb[len(gen):], n, self.a, self.d, self.whiten)
        self.last_metrics = m
        return [float(x) for x in r.cpu()]


def strided_records(token_docs, stride=8, context_length=8, generate_max_len=8, min_completion_prefix=0,
                    bos_token_id=None):
    """Anchor records for strided EBFT from tokenised documents: ``prompt_ids`` = the
    ``context_length`` tokens before the anchor (BOS-prefixed when given), ``ground_truth`` = the
    ``generate_max_len`` tokens after it. Anchors need a full-length continuation."""
    recs = []
    for doc in token_docs:
        doc = [int(t) for t in doc]
        first = max(1, context_length if min_completion_prefix <= 0 else min_completion_prefix)
        for a in range(first, len(doc) - generate_max_len + 1, max(1, stride)):
            ctx = doc[max(0, a - context_length):a]
            if bos_token_id is not None and (not ctx or ctx[0] != bos_token_id):
                ctx = [bos_token_id] + ctx
            recs.append({"prompt_ids": ctx, "ground_truth": doc[a:a + generate_max_len]})
    return recs


def load_strided_records(cfg, tokenizer):
    """Reads the configured datasets as raw text (``text`` field, or pre-tokenised ``input_ids``)."""
    from ..data.loading import _shard, read_raw

    eb = dict(cfg.get("ebft") or {})
    docs = []
    for d in cfg.get("datasets") or []:
        field = d.get("field") or "text"
        for r in _shard(read_raw(dict(d)), dict(d)):
            if "input_ids" in r:
                docs.append(r["input_ids"])
            else:
                if tokenizer is None:
                    raise ValueError("strided EBFT on text datasets needs a tokenizer")
                docs.append(tokenizer(r[field], add_special_tokens=False)["input_ids"])
    bos = tokenizer.bos_token_id if tokenizer is not None else cfg.get("bos_token_id")
    return strided_records(docs, eb.get("stride") or 8, eb.get("context_length") or 8, eb.get("generate_max_len") or 8,
                           eb.get("min_completion_prefix") or 0, bos)
