"""Small helpers, the counterpart of tips/tensorflow/utils.py:5-38 (cache / make_subgraph / refs)."""
from __future__ import annotations

import functools


def cache(fn):
    """Memoise `fn` on its (hashable) arguments."""
    memo = {}

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        key = (args, tuple(sorted(kwargs.items())))
        if key not in memo:
            memo[key] = fn(*args, **kwargs)
        return memo[key]

    wrapper.cache = memo
    return wrapper


def vars_to_refs(params):
    """Hashable references of parameters (ids), and back."""
    return tuple(id(p) for p in params)


def refs_to_vars(refs, params):
    by_id = {id(p): p for p in params}
    return [by_id[r] for r in refs]
