"""Model zoo. Importing this package registers every model family with :class:`ModelRegistry`."""
from .base import BaseModel, ModelRegistry, WeightMapper  # noqa: F401
from . import gpt  # noqa: F401
from . import qwen3_moe  # noqa: F401
from . import deepseek_v3  # noqa: F401
from . import dit  # noqa: F401
from . import mmdit  # noqa: F401
from . import qwen2_5_vl  # noqa: F401
from . import internvl  # noqa: F401
from . import qwen3_vl_moe  # noqa: F401
from . import vla_flow  # noqa: F401
from . import openvla  # noqa: F401
from . import hf_model  # noqa: F401  (fallback for every other transformers causal LM)


def named_architectures():
    """Built-in architectures that can be instantiated with random weights (no download needed)."""
    out = dict(gpt.ARCHS)
    try:
        from . import qwen3_moe
        out.update(qwen3_moe.ARCHS)
        out.update(deepseek_v3.ARCHS)
        out.update(dit.ARCHS)
        out.update(mmdit.ARCHS)
        out.update(qwen2_5_vl.ARCHS)
        out.update(internvl.ARCHS)
        out.update(qwen3_vl_moe.ARCHS)
        out.update(vla_flow.ARCHS)
        out.update(openvla.ARCHS)
    except ImportError:
        pass
    return out
