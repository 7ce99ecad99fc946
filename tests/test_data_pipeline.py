import json
import os

import numpy as np
import pytest
import torch

from axolotl_b200.data.collator import PackedCollator
from axolotl_b200.data.loading import (TokenizedDataset, add_position_ids, apply_pose, calculate_total_num_steps,
                                       dataset_hash, deduplicate, drop_untrainable, filter_lengths, load_datasets,
                                       split_validation)
from axolotl_b200.data.packing import MultipackBatchSampler, pack_first_fit, pack_sequential
from axolotl_b200.data.synthetic import synthetic_fixed, synthetic_varlen


def _first_fit_reference(lengths, cap, bin_size, group):
    out, base = [], 0
    for g0 in range(0, len(lengths), group):
        bins = []  # [remaining, count]
        for l in lengths[g0:g0 + group]:
            if l > cap or l <= 0:
                out.append(-1)
                continue
            for b, (rem, cnt) in enumerate(bins):
                if rem >= l and cnt < bin_size:
                    bins[b] = [rem - l, cnt + 1]
                    out.append(base + b)
                    break
            else:
                bins.append([cap - l, 1])
                out.append(base + len(bins) - 1)
        base += len(bins)
    return out, base


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_first_fit_matches_reference_algorithm(seed):
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, 700, size=3000).astype(np.int32)
    lens[::97] = 5000  # do not fit
    got, n = pack_first_fit(lens, 2048, bin_size=7, group_size=1000)
    ref, nref = _first_fit_reference(lens.tolist(), 2048, 7, 1000)
    assert n == nref and got.tolist() == ref
    used = np.zeros(n, dtype=np.int64)
    cnt = np.zeros(n, dtype=np.int64)
    for l, b in zip(lens, got):
        if b >= 0:
            used[b] += l
            cnt[b] += 1
    assert used.max() <= 2048 and cnt.max() <= 7


def test_sequential_packing_preserves_order():
    lens = np.array([500, 600, 1000, 100, 2048, 1, 3000, 5], dtype=np.int32)
    got, n = pack_sequential(lens, 2048, 200)
    assert got.tolist() == [0, 0, 1, 1, 2, 3, -1, 3] and n == 4


def test_sampler_geometry_and_rank_dealing():
    ds = synthetic_varlen(400, 64, 512, seed=0)
    one_bin = MultipackBatchSampler(ds.lengths, 1024, 2, real_batches=False, seed=3)
    real = MultipackBatchSampler(ds.lengths, 1024, 2, real_batches=True, seed=3)
    b1, b2 = one_bin.all_batches(), real.all_batches()
    assert all(len(b) == 1 for b in b1) and all(len(b) == 2 for b in b2)
    assert all(sum(ds.lengths[i] for i in bins[0]) <= 2048 for bins in b1)
    assert all(sum(ds.lengths[i] for i in bin_) <= 1024 for bins in b2 for bin_ in bins)
    assert 0.8 < real.efficiency() <= 1.0
    r0 = list(MultipackBatchSampler(ds.lengths, 1024, 2, real_batches=True, seed=3, rank=0, world_size=2))
    r1 = list(MultipackBatchSampler(ds.lengths, 1024, 2, real_batches=True, seed=3, rank=1, world_size=2))
    assert len(r0) == len(r1) == len(b2) // 2
    assert r0[0] == b2[0] and r1[0] == b2[1]
    # a different epoch reshuffles
    real.set_epoch(1)
    assert real.all_batches() != b2


def test_packed_collator_layout():
    ds = synthetic_varlen(4, 10, 30, mask_prefix_frac=0.25, seed=1)
    out = PackedCollator(pad_token_id=7, pad_to_multiple_of=64)([[ds[0], ds[1]], [ds[2]]])
    ids, lab, pos = out["input_ids"], out["labels"], out["position_ids"]
    assert ids.shape == (2, 64) and ids.shape == lab.shape == pos.shape
    n0, n1 = len(ds[0]["input_ids"]), len(ds[1]["input_ids"])
    assert pos[0, :n0].tolist() == list(range(n0)) and pos[0, n0:n0 + n1].tolist() == list(range(n1))
    # the pad tail looks like one more document and carries ignored labels
    assert pos[0, n0 + n1:].tolist() == list(range(64 - n0 - n1))
    assert (lab[0, n0 + n1:] == -100).all() and (ids[0, n0 + n1:] == 7).all()
    cu = out["cu_seqlens"].tolist()
    assert cu[:4] == [0, n0, n0 + n1, 64] and cu[-1] == 128
    fixed = PackedCollator(sequence_len=256, pad_to_sequence_len=True)([[ds[0]]])
    assert fixed["input_ids"].shape == (1, 256)


def test_synthetic_fixed_matches_contract():
    d = synthetic_fixed(5, 33, 100, 200, seed=4)
    assert len(d) == 5 and all(len(r["input_ids"]) == 33 for r in d.rows)
    assert all((r["input_ids"] >= 100).all() and (r["input_ids"] < 200).all() for r in d.rows)
    assert all((r["labels"] == r["input_ids"]).all() for r in d.rows)


def test_ragged_dataset_processing(tmp_path):
    rows = [{"input_ids": list(range(1, 1 + n)), "labels": ([-100] * n if n == 6 else list(range(1, 1 + n)))}
            for n in (5, 6, 40, 5, 3)]
    d = TokenizedDataset.from_rows(rows)
    assert d.lengths.tolist() == [5, 6, 40, 5, 3]
    d2 = filter_lengths(d, 32)
    assert d2.lengths.tolist() == [5, 6, 5, 3]
    d3 = drop_untrainable(d2)
    assert d3.lengths.tolist() == [5, 5, 3]
    d4 = deduplicate(d3)
    assert d4.lengths.tolist() == [5, 3]
    add_position_ids(d4)
    assert d4[0]["position_ids"].tolist() == [0, 1, 2, 3, 4]
    with pytest.raises(ValueError):
        filter_lengths(d, 32, strategy="raise")
    t = filter_lengths(d, 32, strategy="truncate")
    assert t.lengths.tolist() == [5, 6, 32, 5, 3]
    d4.save(str(tmp_path / "c"))
    back = TokenizedDataset.load(str(tmp_path / "c"))
    assert back.input_ids.tolist() == d4.input_ids.tolist() and back.position_ids.tolist() == d4.position_ids.tolist()
    tr, ev = split_validation(d, 0.4, seed=1)
    assert len(tr) == 3 and len(ev) == 2
    p = apply_pose(TokenizedDataset.from_rows(rows[:1] * 3), 64, num_chunks=2, seed=0)
    for i in range(3):
        pos = p[i]["position_ids"]
        assert (np.diff(pos) >= 1).all() and pos[-1] < 64


def test_dataset_hash_depends_on_relevant_keys():
    base = {"sequence_len": 512, "seed": 1}
    ds = [{"path": "a.jsonl", "type": "alpaca"}]
    h = dataset_hash(base, ds, "tok")
    assert h == dataset_hash(dict(base), [dict(ds[0])], "tok")
    assert h != dataset_hash({**base, "sequence_len": 1024}, ds, "tok")
    assert h != dataset_hash(base, [{**ds[0], "type": "completion"}], "tok")
    assert h != dataset_hash(base, ds, "other-tok")
    assert h == dataset_hash({**base, "learning_rate": 3.0}, ds, "tok")


def test_load_datasets_cache_and_step_count(tmp_path):
    cfg = {"datasets": [{"type": "_synthetic", "length": 100, "min_length": 50, "max_length": 400, "seed": 0}],
           "sequence_len": 512, "sample_packing": True, "multipack_real_batches": True, "micro_batch_size": 2,
           "batch_size": 4, "gradient_accumulation_steps": 2, "num_epochs": 1, "dataset_prepared_path": str(tmp_path / "prep"),
           "seed": 0, "world_size": 1}
    meta = load_datasets(cfg)
    assert len(meta.train) == 100 and meta.total_num_steps > 0
    sub = os.listdir(tmp_path / "prep")
    assert len(sub) == 1 and os.path.exists(tmp_path / "prep" / sub[0] / "data.npz")
    again = load_datasets(cfg)
    assert again.train.input_ids.tolist() == meta.train.input_ids.tolist()
    assert calculate_total_num_steps({**cfg, "max_steps": 7}, meta.train) == 7
    assert 0 < cfg["sample_packing_eff_est"] <= 1


def test_jsonl_alpaca_pipeline_with_word_tokenizer(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from transformers import PreTrainedTokenizerFast

    words = ["<s>", "</s>", "<unk>", "<pad>"] + [w for w in ("Below is an instruction that describes a task . Write a response "
             "appropriately completes the request ### Instruction: Response: add two numbers four paired with input provides "
             "further context Input: 2 + 2").split()]
    vocab = {w: i for i, w in enumerate(dict.fromkeys(words))}
    t = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    t.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=t, bos_token="<s>", eos_token="</s>", unk_token="<unk>", pad_token="<pad>")
    f = tmp_path / "d.jsonl"
    f.write_text(json.dumps({"instruction": "add two numbers", "input": "2 + 2", "output": "four"}) + "\n" +
                 json.dumps({"instruction": "add two numbers", "input": "", "output": "four"}) + "\n")
    cfg = {"datasets": [{"path": str(f), "type": "alpaca"}], "sequence_len": 128, "dataset_prepared_path": str(tmp_path / "p"),
           "seed": 0, "micro_batch_size": 1, "batch_size": 1, "num_epochs": 1, "world_size": 1}
    meta = load_datasets(cfg, tokenizer=tok)
    assert len(meta.train) == 2
    row = meta.train[0]
    assert row["input_ids"][0] == tok.bos_token_id and row["input_ids"][-1] == tok.eos_token_id
    trainable = row["labels"][row["labels"] != -100]
    assert trainable.tolist() == [vocab["four"], tok.eos_token_id]      # only the response is trained
    cfg2 = {**cfg, "train_on_inputs": True, "dataset_prepared_path": str(tmp_path / "p2")}
    row2 = load_datasets(cfg2, tokenizer=tok).train[0]
    assert (row2["labels"] == row2["input_ids"]).all()


def test_streaming_packed_batches(tmp_path):
    """Lazy jsonl source -> on-the-fly tokenisation -> buffered packing; ranks see disjoint rows."""
    import json

    from axolotl_b200.data.streaming import StreamingPackedBatches

    class Tok:
        bos_token_id, eos_token_id, pad_token_id = 1, 2, 0

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [3 + (ord(c) % 50) for c in text]}

    p = tmp_path / "c.jsonl"
    with open(p, "w") as fh:
        for i in range(200):
            fh.write(json.dumps({"text": "x" * (5 + (i * 7) % 40) + str(i)}) + "\n")
    cfg = {"sequence_len": 128, "micro_batch_size": 2, "pretrain_multipack_buffer_size": 50, "sample_packing": True,
           "pad_to_sequence_len": True, "seed": 1}
    seen = []
    for rank in range(2):
        it = StreamingPackedBatches(cfg, [{"path": str(p), "type": "pretrain"}], Tok(), rank, 2)
        n_tok = 0
        batches = list(it(0))
        assert batches
        for b in batches:
            assert b["input_ids"].shape == (2, 128)
            pos = b["position_ids"]
            assert int((pos == 0).sum()) >= 2            # several documents per row
            lab = b["labels"]
            n_tok += int((lab != -100).sum())
            assert int((b["input_ids"][lab != -100] == 2).sum()) >= 2     # EOS ends every document
        seen.append(n_tok)
    # every row is consumed at most once across the two ranks; only a last incomplete micro-batch
    # (fewer than micro_batch_size bins) may be dropped per rank
    total = sum(5 + (i * 7) % 40 + len(str(i)) + 2 for i in range(200))
    assert 0 <= total - sum(seen) < 2 * 128
