"""A stand-in ``paddle`` module that forwards to torch, so that the reference's own Python code (quantisers,
launchers, adapter, window search, kmeans orchestration) can be EXECUTED by the fixture generator on a machine
where Paddle cannot be installed.  The reference was machine-translated from PyTorch (paddle_utils.py:3-4) and
calls Paddle through a torch-compatible surface (``dim=``, ``device=``, ``.to``, ``.clamp``, ``paddle.compat.*``),
which is what makes a thin forwarder sufficient.  It is used by make_golden.py only; nothing in the library or its
tests imports it.

Every name is forwarded to the torch function of the same meaning.  TWO Paddle semantics are assumptions of this
shim and therefore of every fixture generated through it (they cannot be checked here):

1. ``paddle.round`` rounds halves AWAY from zero (Paddle's documented behaviour); ``torch.round`` rounds halves to
   even, so the shim implements sign(x) * floor(|x| + 0.5).
2. Binary arithmetic between a 16-bit tensor and an fp32 tensor (``x_bf16 / scale_fp32``) promotes to fp32, as
   torch does.

Two substitutions serve the CPU execution and do not touch arithmetic: ``.cuda()`` / ``.place`` / ``device=`` keep
tensors on the CPU, and ``paddle.device.cuda.*`` report one device and do nothing.
"""
import sys
import types

import torch


class _NamedDtype:
    def __init__(self, name):
        self.name = name

    def __str__(self):
        return self.name


def _round_half_away(x):
    return torch.sign(x) * torch.floor(torch.abs(x) + 0.5)


def _two_or_reduce(fn_pair, fn_reduce):
    def f(a, b=None):
        return fn_reduce(a) if b is None else fn_pair(a, b)
    return f


def _dev(kwargs):
    kwargs.pop("device", None)
    return kwargs


def _factory(fn):
    def f(*args, **kwargs):
        return fn(*args, **_dev(kwargs))
    return f


def _zeros_like(x, dtype=None, **kwargs):
    return torch.zeros_like(x, dtype=dtype)


def _bincount(x, weights=None, minlength=0):
    return torch.bincount(x, weights=weights, minlength=minlength)


def _to(self, *args, **kwargs):
    """Tensor.to that ignores devices (a paddle Place or a device string) and keeps dtype conversions."""
    dtype = kwargs.get("dtype")
    for a in args:
        if isinstance(a, torch.dtype):
            dtype = a
    return self if dtype is None or dtype == self.dtype else _orig_to(self, dtype)


_orig_to = torch.Tensor.to


def install():
    """Put the stand-in modules into sys.modules and add the few Paddle-only tensor attributes to torch.Tensor."""
    pd = types.ModuleType("paddle")
    pd.float16, pd.float32, pd.float64, pd.bfloat16 = torch.float16, torch.float32, torch.float64, torch.bfloat16
    pd.int32, pd.int64, pd.bool = torch.int32, torch.int64, torch.bool
    # only ever inspected through str() (fake_quant.py:138-146)
    pd.float8_e4m3fn, pd.float8_e5m2 = _NamedDtype("paddle.float8_e4m3fn"), _NamedDtype("paddle.float8_e5m2")
    pd.Tensor, pd.dtype = torch.Tensor, torch.dtype
    pd.tensor = _factory(torch.tensor)
    for name in ("zeros", "ones", "empty", "full", "arange", "rand", "randn"):
        setattr(pd, name, _factory(getattr(torch, name)))
    pd.zeros_like, pd.ones_like = _zeros_like, lambda x, **kw: torch.ones_like(x)
    pd.round = _round_half_away
    pd.clamp = pd.clip = torch.clamp
    for name in ("sign", "abs", "floor", "log2", "where", "tril", "softmax", "index_select", "finfo", "exp2", "sqrt"):
        setattr(pd, name, getattr(torch, name))
    pd.bincount = _bincount
    compat = types.ModuleType("paddle.compat")
    compat.max = _two_or_reduce(torch.maximum, torch.max)
    compat.min = _two_or_reduce(torch.minimum, torch.min)
    compat.pad = torch.nn.functional.pad
    pd.compat = compat
    cuda = types.SimpleNamespace(empty_cache=lambda: None, device_count=lambda: 1, synchronize=lambda: None)
    pd.device = types.SimpleNamespace(cuda=cuda)
    pd.set_device = lambda *a, **k: None
    sys.modules["paddle"] = pd
    sys.modules["paddle.compat"] = compat
    sys.modules["paddle_utils"] = types.ModuleType("paddle_utils")
    # modules the reference imports for logging / plotting / comparisons and never needs on this path
    for name in ("loguru", "matplotlib", "matplotlib.pyplot", "sageattention", "paddleformers"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.logger = types.SimpleNamespace(info=lambda *a, **k: None, warning=lambda *a, **k: None)
            sys.modules[name] = m
    sdpa = types.ModuleType("sqattn.sdpa_attention")      # the single-query branch of the adapter, not exercised
    sdpa.sdpa_attention_forward = None
    sys.modules["sqattn.sdpa_attention"] = sdpa
    T = torch.Tensor
    T.astype = lambda self, dt: _orig_to(self, dt)
    T.place = property(lambda self: self.device)
    T.strides = property(lambda self: self.stride())
    T.cuda = lambda self, *a, **k: self
    T.to = _to
    T._max = lambda self: self.max()
    return pd
