"""NumPy-backed stand-in for the small part of ``mlx.core`` that the reference's
pure-MLX modules (rotation, codebook, packing, qjl, quantizer, cache) touch.

Test infrastructure only: ``make_golden.py`` puts this directory on ``sys.path``
so the unmodified reference package imports and runs on the CPU, and the
fixtures it writes pin the oracle.  Nothing in the shipped package imports it.

Three properties of MLX are reproduced because results depend on them:

* Python floats become float32 arrays (NumPy would make float64 and promote).
* Slicing yields a value, not a view (``cache._drain_chunk`` takes a slice and
  then shifts the same buffer in place).
* ``mx.array`` is a type usable in ``mx.array | None`` and ``isinstance``.
"""

import numpy as np

float16 = np.float16
float32 = np.float32
uint8 = np.uint8
uint16 = np.uint16
uint32 = np.uint32
int32 = np.int32
int64 = np.int64
bool_ = np.bool_


class array(np.ndarray):
    """ndarray subclass with MLX's value-semantic indexing and float32 default."""

    def __new__(cls, obj, dtype=None):
        if dtype is None and isinstance(obj, float):
            dtype = np.float32
        a = np.array(obj, dtype=dtype)
        if dtype is None and a.dtype == np.float64 and not isinstance(obj, np.ndarray):
            a = a.astype(np.float32)
        return a.view(cls)

    def __getitem__(self, idx):
        out = super().__getitem__(idx)
        if isinstance(out, np.ndarray):
            out = np.array(out, copy=True).view(array)
        return out

    def __setitem__(self, idx, val):
        # Write through a plain view: with __getitem__ overridden to copy, NumPy's own
        # slice assignment on the subclass would land in a temporary.
        np.ndarray.__setitem__(self.view(np.ndarray), idx, np.asarray(val))

    def astype(self, dtype, *a, **k):
        return np.ndarray.astype(self, dtype, *a, **k).view(array)

    def item(self):
        return np.ndarray.item(self)


def _wrap(x):
    return x.view(array) if isinstance(x, np.ndarray) else array(x)


def maximum(a, b):
    return _wrap(np.maximum(a, b))


def sum(a, axis=None):  # noqa: A001 - mirrors mx.sum
    a = np.asarray(a)
    # MLX keeps the input integer type when summing; NumPy widens to 64-bit.
    dt = a.dtype if a.dtype.kind in "ui" else None
    return _wrap(np.sum(a, axis=axis, dtype=dt))


def mean(a, axis=None):
    return _wrap(np.mean(np.asarray(a), axis=axis, dtype=np.float32))


def max(a, axis=None):  # noqa: A001
    return _wrap(np.max(np.asarray(a), axis=axis))


def abs(a):  # noqa: A001
    return _wrap(np.abs(np.asarray(a)))


def stack(xs, axis=0):
    return _wrap(np.stack([np.asarray(x) for x in xs], axis=axis))


def concatenate(xs, axis=0):
    return _wrap(np.concatenate([np.asarray(x) for x in xs], axis=axis))


def where(c, a, b):
    return _wrap(np.where(np.asarray(c), np.asarray(a), np.asarray(b)))


def zeros(shape, dtype=np.float32):
    return _wrap(np.zeros(shape, dtype=dtype))


def ones(shape, dtype=np.float32):
    return _wrap(np.ones(shape, dtype=dtype))


def full(shape, v, dtype=np.float32):
    return _wrap(np.full(shape, v, dtype=dtype))


def diag(a):
    return _wrap(np.diag(np.asarray(a)))


def eval(*a):  # noqa: A001 - MLX's graph materialisation; nothing is lazy here
    return None


class _Linalg:
    @staticmethod
    def norm(x, axis=None):
        x = np.asarray(x)
        return _wrap(np.sqrt(np.sum(x * x, axis=axis, dtype=x.dtype)))


linalg = _Linalg()


class _MetalKernelStub:
    def __call__(self, *a, **k):
        raise RuntimeError("Metal is unavailable on this box")


class _Fast:
    @staticmethod
    def metal_kernel(**kw):
        return _MetalKernelStub()


fast = _Fast()
