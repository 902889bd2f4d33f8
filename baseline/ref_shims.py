"""Import-time stand-ins for packages the reference imports at module scope but that are not installed here.

The reference tree under ``baseline/_ref`` stays unmodified. Its modules import ``strenum``, ``redis``,
``torchao.float8``, ``diffusers`` (and a few optional accelerators) at import time even on code paths that never
call them (bf16 training of a dense decoder needs none of them). ``install()`` registers a meta-path finder that
serves empty placeholder modules for exactly those absent top-level packages; any attribute read from a placeholder
yields an inert class, so ``from diffusers import DiffusionPipeline`` succeeds and nothing else changes. A package
that IS installed is never shadowed. Calling into a placeholder raises, so a path that really needs the package
fails loudly instead of computing something else. Two names are real stand-ins because the bf16 dense path calls them:
``strenum.StrEnum`` (= ``enum.StrEnum``) and ``accelerate.init_on_device`` (a context manager that creates
parameters on the meta device, restated below).
"""
from __future__ import annotations

import contextlib
import enum
import importlib.abc
import importlib.machinery
import importlib.util
import os
import sys
import types

ABSENT_OK = ("strenum", "redis", "torchao", "diffusers", "qwen_vl_utils", "accelerate", "peft", "boto3", "botocore")


def _refuse(qualname: str):
    def fn(*a, **k):
        raise RuntimeError(f"{qualname} is a placeholder for a package that is not installed on this machine")
    fn.__qualname__ = fn.__name__ = qualname.rsplit(".", 1)[-1]
    return fn


class _InertMeta(type):
    def __getattr__(cls, name: str):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        return _refuse(f"{cls.__module__}.{cls.__qualname__}.{name}")


class _Inert(metaclass=_InertMeta):
    """What an attribute of a placeholder module evaluates to: subclassable, but not usable."""

    def __init__(self, *a, **k):
        raise RuntimeError(f"{type(self).__module__}.{type(self).__qualname__} is a placeholder for a package that is "
                           "not installed on this machine")

    def __init_subclass__(cls, **k):
        pass

    @classmethod
    def __class_getitem__(cls, item):
        return cls


class _Placeholder(types.ModuleType):
    def __getattr__(self, name: str):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        if name[:1].islower() and name not in ("float8",):
            # lower-case names are mostly sub-modules or functions: a callable sub-module placeholder covers both
            sub = _Callable(f"{self.__name__}.{name}")
            sub.__path__ = []
            sub.__spec__ = importlib.machinery.ModuleSpec(sub.__name__, _FINDER, is_package=True)
            sys.modules.setdefault(sub.__name__, sub)
            setattr(self, name, sub)
            return sub
        cls = type(name, (_Inert,), {"__module__": self.__name__})
        setattr(self, name, cls)
        return cls


class _Callable(_Placeholder):
    def __call__(self, *a, **k):
        raise RuntimeError(f"{self.__name__} is a placeholder for a package that is not installed on this machine")


@contextlib.contextmanager
def init_on_device(device, include_buffers: bool = False):
    """Working stand-in for ``accelerate.init_on_device`` (the one function of that package the reference calls when
    it builds a model, cosmos_rl/policy/model/base.py:706): inside the context every parameter a module registers
    is moved to ``device`` (``"meta"`` = no storage), and buffers too when ``include_buffers``."""
    import torch
    from torch import nn
    device = torch.device(device)
    reg_param, reg_buffer = nn.Module.register_parameter, nn.Module.register_buffer

    def register_parameter(module, name, param):
        reg_param(module, name, param)
        if param is not None:
            cur = module._parameters[name]
            extra = dict(cur.__dict__)
            extra["requires_grad"] = param.requires_grad
            module._parameters[name] = type(cur)(cur.to(device), **extra)

    def register_buffer(module, name, buffer, persistent=True):
        reg_buffer(module, name, buffer, persistent=persistent)
        if buffer is not None:
            module._buffers[name] = module._buffers[name].to(device)

    nn.Module.register_parameter = register_parameter
    if include_buffers:
        nn.Module.register_buffer = register_buffer
    try:
        yield
    finally:
        nn.Module.register_parameter = reg_param
        nn.Module.register_buffer = reg_buffer


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def __init__(self):
        self.served = set()

    @staticmethod
    def _asked_by_reference() -> bool:
        """Only imports written in the reference's own files are served: third-party packages that probe for an
        optional dependency (``importlib.util.find_spec("torchao")``) must keep seeing it as absent."""
        f = sys._getframe(2)
        while f is not None:
            fn = f.f_code.co_filename
            if "importlib" not in fn and not fn.startswith("<frozen"):
                return os.sep + "_ref" + os.sep in fn
            f = f.f_back
        return False

    def find_spec(self, fullname, path=None, target=None):
        top = fullname.split(".")[0]
        if top not in ABSENT_OK or not (top in self.served or self._asked_by_reference()):
            return None
        if top not in self.served:
            # shadow nothing that exists
            for f in sys.meta_path:
                if f is self:
                    continue
                try:
                    if f.find_spec(top, None) is not None:
                        return None
                except Exception:
                    continue
            self.served.add(top)
        return importlib.machinery.ModuleSpec(fullname, self, is_package=True)

    def create_module(self, spec):
        m = _Callable(spec.name)
        m.__path__ = []
        if spec.name == "strenum":
            m.StrEnum = enum.StrEnum
        if spec.name == "accelerate":
            m.init_on_device = init_on_device
            m.init_empty_weights = lambda include_buffers=False: init_on_device("meta", include_buffers)
        return m

    def exec_module(self, module):
        pass


_FINDER = _Finder()


def install() -> _Finder:
    # availability probes of installed libraries are cached on first use: take them before any placeholder exists
    try:
        from transformers.utils import import_utils as _iu
        for probe in ("is_torchao_available", "is_peft_available", "is_accelerate_available"):
            fn = getattr(_iu, probe, None)
            if fn is not None:
                try:
                    fn()
                except Exception:
                    pass
    except Exception:
        pass
    if _FINDER not in sys.meta_path:
        sys.meta_path.append(_FINDER)      # last: only reached when no real finder knows the name
    return _FINDER
