"""``Module``, ``Parameter``, ``Linear``, ``Sequential``: what ``quantize_``
and ``load_quantized_`` walk and rewrite (python/grilly/nn/modules/layers.py:33-57,
python/grilly/nn/parameter.py:8-23)."""
from __future__ import annotations

import math
from collections import OrderedDict

import numpy as np

from .. import Tensor, _require_tensor, from_numpy
from . import functional as F

_init_rng = np.random.default_rng(0)


class Parameter(Tensor):
    """A tensor that a ``Module`` registers when it is assigned as an
    attribute. Shares data with the tensor it wraps."""

    __slots__ = ()

    def __new__(cls, data=None, requires_grad: bool = False):
        core = _require_tensor("data", data)._t
        return Tensor._wrap.__func__(cls, core)

    def __init__(self, data=None, requires_grad: bool = False) -> None:
        pass

    def __repr__(self) -> str:
        return "Parameter containing:\n" + super().__repr__()


class Module:
    def __init__(self) -> None:
        object.__setattr__(self, "_parameters", OrderedDict())
        object.__setattr__(self, "_modules", OrderedDict())

    def __setattr__(self, name, value) -> None:
        params, mods = self.__dict__.get("_parameters"), self.__dict__.get("_modules")
        if params is None:
            raise AttributeError("cannot assign before Module.__init__() call")
        if isinstance(value, Parameter):
            mods.pop(name, None)
            self.__dict__.pop(name, None)
            params[name] = value
        elif isinstance(value, Module):
            params.pop(name, None)
            self.__dict__.pop(name, None)
            mods[name] = value
        elif name in params:
            if value is not None:
                raise TypeError(f"cannot assign '{type(value).__name__}' as parameter '{name}' (nn.Parameter or None expected)")
            params[name] = None
        else:
            object.__setattr__(self, name, value)

    def __getattr__(self, name):
        d = self.__dict__
        if "_parameters" in d and name in d["_parameters"]:
            return d["_parameters"][name]
        if "_modules" in d and name in d["_modules"]:
            return d["_modules"][name]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{name}'")

    def register_parameter(self, name, param) -> None:
        self._parameters[name] = param

    def named_modules(self, prefix: str = ""):
        yield prefix, self
        for name, mod in self._modules.items():
            yield from mod.named_modules(f"{prefix}.{name}" if prefix else name)

    def modules(self):
        for _, m in self.named_modules():
            yield m

    def named_parameters(self, prefix: str = ""):
        for mname, mod in self.named_modules(prefix):
            for pname, p in mod._parameters.items():
                if p is not None:
                    yield (f"{mname}.{pname}" if mname else pname), p

    def parameters(self):
        for _, p in self.named_parameters():
            yield p

    def get_submodule(self, target: str) -> "Module":
        mod = self
        for part in target.split(".") if target else []:
            mod = mod._modules[part]
        return mod

    def state_dict(self, keep_vars: bool = False) -> "OrderedDict":
        """Names to tensors. A quantized weight appears dequantized unless
        ``keep_vars`` (python/grilly/infer/quantization.py:28-31;
        tests/python/test_load_quantized.py:145-160)."""
        out = OrderedDict()
        for name, p in self.named_parameters():
            out[name] = p if keep_vars or not hasattr(p, "dequantize") else p.dequantize()
        return out

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        own = dict(self.named_parameters())
        missing = [k for k in own if k not in state_dict]
        unexpected = [k for k in state_dict if k not in own]
        errors = []
        for key, value in state_dict.items():
            if key not in own:
                continue
            if tuple(value.shape) != tuple(own[key].shape):
                errors.append(f"size mismatch for {key}: copying a param with shape {list(value.shape)} from "
                              f"checkpoint, the shape in current model is {list(own[key].shape)}.")
                continue
            owner, _, attr = key.rpartition(".")
            setattr(self.get_submodule(owner), attr, Parameter(value))
        if strict:
            if missing:
                errors.insert(0, "Missing key(s) in state_dict: " + ", ".join(f'"{k}"' for k in missing))
            if unexpected:
                errors.insert(0, "Unexpected key(s) in state_dict: " + ", ".join(f'"{k}"' for k in unexpected))
        if errors:
            raise RuntimeError(f"Error(s) in loading state_dict for {type(self).__name__}:\n\t" + "\n\t".join(errors))
        return missing, unexpected

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def extra_repr(self) -> str:
        return ""

    def __repr__(self) -> str:
        lines = [f"  ({k}): " + repr(m).replace("\n", "\n  ") for k, m in self._modules.items()]
        head = f"{type(self).__name__}({self.extra_repr()}"
        return head + ")" if not lines else head + "\n" + "\n".join(lines) + "\n)"


class Linear(Module):
    """``y = x W^T + b``; weight (out_features, in_features), kaiming-uniform
    with bound 1/sqrt(in_features) like torch's, drawn from numpy."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        from .. import _resolve_device
        _resolve_device(device)
        self.in_features, self.out_features = in_features, out_features
        bound = 1 / math.sqrt(in_features) if in_features > 0 else 0
        self.weight = Parameter(from_numpy(_init_rng.uniform(-bound, bound, (out_features, in_features)).astype(np.float32), persistent=True))
        if bias:
            self.bias = Parameter(from_numpy(_init_rng.uniform(-bound, bound, out_features).astype(np.float32), persistent=True))
        else:
            self.register_parameter("bias", None)

    def forward(self, input):
        return F.linear(input, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class Sequential(Module):
    def __init__(self, *mods) -> None:
        super().__init__()
        for i, m in enumerate(mods):
            setattr(self, str(i), m)

    def __getitem__(self, i: int) -> Module:
        return list(self._modules.values())[i]

    def __len__(self) -> int:
        return len(self._modules)

    def forward(self, x):
        for m in self._modules.values():
            x = m(x)
        return x
