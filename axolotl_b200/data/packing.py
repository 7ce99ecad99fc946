"""Multipack sample packing.

Semantics follow the reference sampler (src/axolotl/utils/samplers/multipack.py:60-473 and
src/axolotl/core/trainers/base.py:141-249): samples are visited in sampler order (shuffled with
the epoch seed, or sequential), packed first-fit into bins of ``batch_max_len`` tokens holding at
most ``bin_size`` samples, independently per group of ``group_size`` samples; a batch is a list of
bins. ``real_batches=True`` yields ``batch_size`` bins of ``sequence_len``; the default yields ONE
bin of ``batch_size * sequence_len`` per batch. The batch list is identical on every rank and is
dealt out round-robin; its length is agreed across ranks (minimum). The bin packing itself runs in
the native host library instead of numba.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from ..ops import _lib


def pack_first_fit(lengths, capacity, bin_size=200, group_size=100_000):
    """bin index per sample (-1 = does not fit) and number of bins."""
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    out = np.empty(len(lengths), dtype=np.int32)
    n = _lib.host_lib().axb_pack_first_fit(lengths.ctypes.data, len(lengths), int(capacity), int(bin_size),
                                           int(group_size), out.ctypes.data)
    return out, n


def pack_sequential(lengths, capacity, bin_size=200):
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    out = np.empty(len(lengths), dtype=np.int32)
    n = _lib.host_lib().axb_pack_sequential(lengths.ctypes.data, len(lengths), int(capacity), int(bin_size),
                                            out.ctypes.data)
    return out, n


def bins_from_assignment(order, bin_of, n_bins):
    """list of bins, each a list of dataset indices in visiting order."""
    bins = [[] for _ in range(n_bins)]
    for idx, b in zip(order, bin_of):
        if b >= 0:
            bins[b].append(int(idx))
    return [b for b in bins if b]


class MultipackBatchSampler:
    def __init__(self, lengths, batch_max_len, batch_size=1, *, real_batches=False, bin_size=200,
                 group_size=100_000, sequential=False, shuffle=True, seed=0, drop_last=True,
                 rank=0, world_size=1, len_agree_fn=None):
        self.lengths = np.asarray(lengths, dtype=np.int32)
        self.batch_size = batch_size
        self.real_batches = real_batches
        self.batch_max_len = batch_max_len if real_batches else batch_max_len * batch_size
        self.bins_per_batch = batch_size if real_batches else 1
        self.bin_size, self.group_size = bin_size, group_size
        self.sequential, self.shuffle, self.seed = sequential, shuffle, seed
        self.drop_last = drop_last
        self.rank, self.world_size = rank, world_size
        self.epoch = 0
        self.len_agree_fn = len_agree_fn
        self._eff = None
        self._len = None

    def set_epoch(self, epoch):
        self.epoch = epoch
        self._len = None

    def _order(self):
        n = len(self.lengths)
        if self.shuffle and not self.sequential:
            return np.random.default_rng(self.seed + self.epoch).permutation(n)
        return np.arange(n)

    def all_batches(self):
        """The global batch list (same on every rank)."""
        order = self._order()
        lens = self.lengths[order]
        if self.sequential:
            bin_of, n = pack_sequential(lens, self.batch_max_len, self.bin_size)
        else:
            bin_of, n = pack_first_fit(lens, self.batch_max_len, self.bin_size, self.group_size)
        bins = bins_from_assignment(order, bin_of, n)
        used = sum(int(self.lengths[i]) for b in bins for i in b)
        self._eff = used / max(1, len(bins) * self.batch_max_len)
        k = self.bins_per_batch
        batches = [bins[i:i + k] for i in range(0, len(bins), k)]
        if self.drop_last and batches and len(batches[-1]) < k:
            batches.pop()
        return batches

    def efficiency(self):
        if self._eff is None:
            self.all_batches()
        return self._eff

    def __iter__(self):
        batches = self.all_batches()
        n = len(self)
        mine = batches[self.rank::self.world_size][:n]
        return iter(mine)

    def __len__(self):
        if self._len is None:
            per_rank = len(self.all_batches()) // self.world_size
            if self.len_agree_fn is not None:
                per_rank = int(self.len_agree_fn(per_rank))
            self._len = per_rank
        return self._len


def estimate_total_steps(num_batches_per_rank, micro_batch_size, batch_size_per_rank_step, num_epochs,
                         drop_last=True):
    """len(dataloader) * micro_batch_size // batch_size * epochs (minus ceil(epochs) with drop_last)
    as in src/axolotl/utils/trainer.py:494-503."""
    steps = int(num_batches_per_rank * micro_batch_size // batch_size_per_rank_step * num_epochs)
    if drop_last:
        steps -= int(math.ceil(num_epochs))
    return max(steps, 0)
