"""A numpy stand-in for the handful of JAX calls the reference's quantize/dequantize use.

JAX is not installed where the golden vectors are generated, so `make_golden.py` registers these
modules under the names `jax`, `jax.numpy`, `jax.scipy`, `jax.lax` and `optax` and then imports the
reference's OWN rptc.py / rptc_lite.py unmodified.  Only what those two files touch at import time
and inside quantize / dequantize is provided; semantics follow JAX's defaults (32-bit integers that
wrap, 32-bit floats, functional `.at[...]` updates, lax.scan stacking its per-step outputs).
"""
from __future__ import annotations

import sys
import types

import numpy as np


class Arr(np.ndarray):
    @property
    def at(self):
        return _At(self)


class _At:
    def __init__(self, a):
        self.a = a

    def __getitem__(self, idx):
        return _AtIdx(self.a, idx)


class _AtIdx:
    def __init__(self, a, idx):
        self.a, self.idx = a, idx

    def set(self, v):
        out = np.array(self.a, copy=True)
        out[self.idx] = np.asarray(v).astype(out.dtype)
        return out.view(Arr)

    def add(self, v):
        out = np.array(self.a, copy=True)
        with np.errstate(over="ignore"):
            out[self.idx] = (out[self.idx].astype(np.int64) + np.asarray(v).astype(np.int64)).astype(out.dtype) \
                if np.issubdtype(out.dtype, np.integer) else out[self.idx] + v
        return out.view(Arr)


def _wrap(x):
    if isinstance(x, np.ndarray):
        return x.view(Arr)
    return x


def _dtype(dt, default):
    if dt is None:
        return default
    if dt is int:
        return np.int32
    if dt is float:
        return np.float32
    return dt


jnp = types.ModuleType("jax.numpy")
jnp.newaxis = None
jnp.inf = np.float32(np.inf)
jnp.int32 = np.int32
jnp.float32 = np.float32
jnp.iinfo = np.iinfo


def _arange(*a, dtype=None):
    return _wrap(np.arange(*a, dtype=_dtype(dtype, np.int32)))


def _full(shape, v, dtype=None):
    return _wrap(np.full(shape, v, dtype=_dtype(dtype, np.float32 if isinstance(v, (float, np.floating)) else np.int32)))


jnp.arange = _arange
jnp.full = _full
jnp.empty = lambda shape, dtype=None: _wrap(np.zeros(shape, dtype=_dtype(dtype, np.float32)))
jnp.zeros = lambda shape, dtype=None: _wrap(np.zeros(shape, dtype=_dtype(dtype, np.float32)))
jnp.ones = lambda shape, dtype=None: _wrap(np.ones(shape, dtype=_dtype(dtype, np.float32)))
jnp.eye = lambda n, dtype=None: _wrap(np.eye(n, dtype=_dtype(dtype, np.float32)))
jnp.array = lambda x, dtype=None: _wrap(np.array(x, dtype=dtype))
jnp.asarray = jnp.array
jnp.argmin = lambda a, axis=None: _wrap(np.asarray(np.argmin(a, axis=axis)).astype(np.int32))
jnp.min = lambda a, axis=None: _wrap(np.min(a, axis=axis))
jnp.sum = lambda a, axis=None, keepdims=False: _wrap(np.sum(a, axis=axis, keepdims=keepdims))
jnp.mean = lambda a, axis=None, keepdims=False: _wrap(np.mean(a, axis=axis, keepdims=keepdims))
jnp.repeat = lambda a, r: _wrap(np.repeat(a, r))
jnp.flipud = lambda a: _wrap(np.flipud(a))
jnp.reshape = lambda a, s: _wrap(np.reshape(a, s))
jnp.ravel = lambda a: _wrap(np.ravel(a))
jnp.sqrt = np.sqrt
jnp.log2 = np.log2
jnp.bincount = lambda a, length=None: _wrap(np.bincount(a, minlength=length))

jnp.exp = np.exp
jnp.log = np.log
jnp.diag = lambda a: _wrap(np.diag(a))
jnp.sort = lambda a, axis=-1: _wrap(np.sort(a, axis=axis))
jnp.interp = lambda x, xp, fp: _wrap(np.interp(x, xp, fp).astype(np.float32))

lax = types.ModuleType("jax.lax")


def _tree_map(f, t):
    if isinstance(t, tuple):
        return tuple(_tree_map(f, x) for x in t)
    return f(t)


def _scan(f, init, xs, length=None):
    carry = init
    ys = []
    n = len(xs) if xs is not None else length
    for i in range(n):
        x = xs[i] if xs is not None else None
        carry, y = f(carry, x)
        ys.append(y)
    if ys and ys[0] is not None:
        if isinstance(ys[0], tuple):
            stacked = tuple(_wrap(np.stack([np.asarray(y[k]) for y in ys])) for k in range(len(ys[0])))
        else:
            stacked = _wrap(np.stack([np.asarray(y) for y in ys]))
    else:
        stacked = None
    return carry, stacked


def _while_loop(cond, body, init):
    val = init
    while bool(np.all(cond(val))):
        val = body(val)
    return val


lax.scan = _scan
lax.while_loop = _while_loop
lax.map = lambda f, xs: _wrap(np.stack([np.asarray(f(x)) for x in xs]))

jax = types.ModuleType("jax")
jax.numpy = jnp
jax.lax = lax
jax.jit = lambda f=None, **kw: f if f is not None else (lambda g: g)
jax.scipy = types.ModuleType("jax.scipy")
jax.random = types.ModuleType("jax.random")
optax = types.ModuleType("optax")


def _vmap(f, in_axes):
    """jax.vmap for in_axes made of None and 0, outputs an array or a tuple of arrays."""
    def mapped(*args):
        n = next(len(a) for a, ax in zip(args, in_axes) if ax == 0)
        outs = [f(*[a[i] if ax == 0 else a for a, ax in zip(args, in_axes)]) for i in range(n)]
        if isinstance(outs[0], tuple):
            return tuple(_wrap(np.stack([np.asarray(o[k]) for o in outs])) for k in range(len(outs[0])))
        return _wrap(np.stack([np.asarray(o) for o in outs]))
    return mapped


# Keys are plain integers here; a permutation is numpy's default_rng(key).permutation -- NOT JAX's
# threefry stream, so only code that is handed the permuted alphabet can be compared with these vectors.
jax.vmap = _vmap
jax.random.PRNGKey = lambda seed: int(seed)
jax.random.fold_in = lambda key, data: int(key) * 1000003 + int(data)
jax.random.permutation = lambda key, a: _wrap(np.asarray(a)[np.random.default_rng(int(key)).permutation(len(a))])


def install() -> None:
    sys.modules.setdefault("jax", jax)
    sys.modules.setdefault("jax.numpy", jnp)
    sys.modules.setdefault("jax.lax", lax)
    sys.modules.setdefault("jax.scipy", jax.scipy)
    sys.modules.setdefault("jax.random", jax.random)
    sys.modules.setdefault("optax", optax)
