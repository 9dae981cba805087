"""Import the reference's own Python package (``lpmm``) on CPU tensors.  TEST INFRASTRUCTURE ONLY.

The reference cannot be imported as shipped in a CPU-only container for two reasons, both worked
around here without touching its files:

* ``lpmm/config.py:4`` imports ``yacs.config.CfgNode``; yacs is not installed.  A minimal
  stand-in with the handful of methods the reference uses (``config.py:7-94,185``) is registered
  as ``yacs.config``.
* ``lpmm/functional.py:4`` imports the CUDA extension ``lpmm.cpp_extension.quantization``.  A CPU
  module with the same two functions is registered under that name; it restates
  ``pack_nonlinear`` / ``unpack_nonlinear`` (``quantization.cc:54-76`` ->
  ``quantization_kernel.cu:430-513, 604-653``) on top of ``oracle/lpmm_oracle.c``.

Used by ``tests/golden/make_python_golden.py`` to produce fixtures and by CPU tests that compare
this repository's restatements with the reference when the checkout is available.  The reference
package shadows the product package of the same name, so only ever call ``load_reference()`` in a
process that does not import the product.
"""
import copy
import os
import sys
import types

import numpy as np


class CfgNode(dict):
    """Just enough of yacs.config.CfgNode for lpmm/config.py."""

    def __init__(self, init_dict=None, key_list=None, new_allowed=False):
        super().__init__()
        self.__dict__["_frozen"] = False
        self.__dict__["_new_allowed"] = new_allowed
        for k, v in (init_dict or {}).items():
            self[k] = CfgNode(v, new_allowed=new_allowed) if isinstance(v, dict) and not isinstance(v, CfgNode) else v

    def __getattr__(self, name):
        if name in self:
            return self[name]
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if self.__dict__["_frozen"]:
            raise AttributeError(f"Attempted to set {name} to {value}, but CfgNode is immutable")
        self[name] = value

    def __str__(self):
        def _indent(s, n):
            lines = s.split("\n")
            return "\n".join([lines[0]] + [(" " * n) + l for l in lines[1:]])

        parts = []
        for k, v in sorted(self.items()):
            sep = "\n" if isinstance(v, CfgNode) else " "
            parts.append(_indent(f"{k}:{sep}{v}", 2))
        return "\n".join(parts)

    def __repr__(self):
        return f"CfgNode({dict.__repr__(self)})"

    def clone(self):
        return copy.deepcopy(self)

    def __deepcopy__(self, memo):
        new = CfgNode(new_allowed=self.__dict__["_new_allowed"])
        for k, v in self.items():
            dict.__setitem__(new, k, copy.deepcopy(v, memo))
        new.__dict__["_frozen"] = self.__dict__["_frozen"]
        return new

    def __reduce__(self):
        return (_rebuild, (dict(self), self.__dict__["_new_allowed"], self.__dict__["_frozen"]))

    def _set_frozen(self, flag):
        self.__dict__["_frozen"] = flag
        for v in self.values():
            if isinstance(v, CfgNode):
                v._set_frozen(flag)

    def defrost(self):
        self._set_frozen(False)

    def freeze(self):
        self._set_frozen(True)

    def is_frozen(self):
        return self.__dict__["_frozen"]

    def merge_from_file(self, path):
        import yaml
        with open(path) as f:
            other = yaml.safe_load(f) or {}
        self._merge(other)

    def _merge(self, other):
        for k, v in other.items():
            if isinstance(v, dict) and isinstance(self.get(k), CfgNode):
                self[k]._merge(v)
            elif isinstance(v, dict):
                dict.__setitem__(self, k, CfgNode(v, new_allowed=True))
            else:
                dict.__setitem__(self, k, v)


def _rebuild(items, new_allowed, frozen):
    n = CfgNode(new_allowed=new_allowed)
    for k, v in items.items():
        dict.__setitem__(n, k, v)
    n.__dict__["_frozen"] = frozen
    return n


def _install_yacs():
    if "yacs.config" in sys.modules:
        return
    yacs = types.ModuleType("yacs")
    cfg = types.ModuleType("yacs.config")
    cfg.CfgNode = CfgNode
    yacs.config = cfg
    sys.modules["yacs"] = yacs
    sys.modules["yacs.config"] = cfg


def _cpu_quantization_module():
    """CPU stand-in for lpmm.cpp_extension.quantization (4 to 8 bits, round-to-nearest only)."""
    import torch
    from . import cpu

    mod = types.ModuleType("lpmm.cpp_extension.quantization")

    def pack_nonlinear(data, qmap, bits, stochastic):
        # quantization.cc:54-63: bits <= 8, data 2-D float, qmap 1-D float
        assert 4 <= bits <= 8 and not stochastic, "the CPU stand-in covers 4 to 8 bits, round-to-nearest only"
        assert data.dim() == 2 and qmap.dim() == 1
        if bits == 4:  # quantization_kernel.cu:596-600
            assert data.shape[1] % 8 == 0  # quantization_kernel.cu:473
            packed = cpu.pack4(data.detach().contiguous().numpy(), qmap.numpy())
        else:
            assert data.shape[1] % 4 == 0  # quantization_kernel.cu:550
            packed = cpu.pack8(data.detach().contiguous().numpy(), qmap.numpy(), bits)
        return torch.from_numpy(packed.view(np.int8))

    def unpack_nonlinear(data, qmap, bits, num_groups, group_size):
        # quantization.cc:65-76
        assert 4 <= bits <= 8 and data.dim() == 1 and data.dtype == torch.int8
        if bits == 4:  # quantization_kernel.cu:700-704
            out = cpu.unpack4(data.contiguous().numpy(), qmap.numpy(), int(num_groups), int(group_size))
        else:
            out = cpu.unpack8(data.contiguous().numpy(), qmap.numpy(), bits, int(num_groups), int(group_size))
        return torch.from_numpy(out)

    mod.pack_nonlinear = pack_nonlinear
    mod.unpack_nonlinear = unpack_nonlinear
    return mod


def load_reference(reference_root=None):
    """Import and return the reference's ``lpmm`` package (CPU only).  ``reference_root``: a directory that
    holds the reference's ``lpmm`` package -- a checkout, or the Python layer that ``oracle/build_ref.py``
    placed under ``oracle/_ref/lpmm_py``; default: the checkout ``build_ref.reference_root()`` finds, else
    that copy."""
    if reference_root is None:
        from . import build_ref
        reference_root = build_ref.reference_root() or (build_ref.PY_OUT if build_ref.have_python() else None)
    if reference_root is None or not os.path.isdir(os.path.join(reference_root, "lpmm")):
        raise FileNotFoundError(f"no reference package at {reference_root}")
    if "lpmm" in sys.modules and not getattr(sys.modules["lpmm"], "__file__", "").startswith(reference_root):
        raise RuntimeError("another package named lpmm is already imported in this process")
    _install_yacs()
    ext_pkg = types.ModuleType("lpmm.cpp_extension")
    ext_pkg.__path__ = []
    quant = _cpu_quantization_module()
    ext_pkg.quantization = quant
    sys.modules["lpmm.cpp_extension"] = ext_pkg
    sys.modules["lpmm.cpp_extension.quantization"] = quant
    if reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    import lpmm  # noqa: E402  (the reference)
    lpmm.cpp_extension = ext_pkg
    return lpmm
