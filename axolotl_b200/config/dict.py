"""Attribute dictionary that returns None for missing keys (the configuration object every layer
reads; same behaviour as the reference's DictDefault, src/axolotl/utils/dict.py)."""
from __future__ import annotations


class DictDefault(dict):
    def __init__(self, *args, **kwargs):
        super().__init__()
        for k, v in dict(*args, **kwargs).items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, dict) and not isinstance(v, DictDefault):
            return DictDefault(v)
        if isinstance(v, list):
            return [DictDefault._wrap(x) for x in v]
        return v

    def __setitem__(self, k, v):
        super().__setitem__(k, self._wrap(v))

    def __getattr__(self, k):
        if k.startswith("__"):
            raise AttributeError(k)
        return self.get(k)

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        self.pop(k, None)

    def __missing__(self, k):
        return None

    def __or__(self, other):
        return DictDefault({**self, **other})

    def to_dict(self):
        def un(v):
            if isinstance(v, DictDefault):
                return {k: un(x) for k, x in v.items()}
            if isinstance(v, list):
                return [un(x) for x in v]
            return v

        return un(self)
