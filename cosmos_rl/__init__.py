"""Import-compatibility alias: ``cosmos_rl.<module>`` resolves to ``cosmos_rl_b200.<module>``.

User entry scripts written for the reference (``from cosmos_rl.launcher.worker_entry import main``,
``from cosmos_rl.dispatcher.data.packer import BaseDataPacker`` ...) run unchanged. Only module paths that exist in
``cosmos_rl_b200`` resolve; nothing of the reference is imported or required.
"""
import importlib
import importlib.abc
import importlib.util
import sys

_TARGET = "cosmos_rl_b200"
# module paths that moved: reference path -> path inside this package
_MOVED = {
    "dispatcher.data.packer": "data.packer",
    "dispatcher.data.packer.base": "data.packer",
    "dispatcher.data.packer.decoder_only_llm_data_packer": "data.packer",
    "policy.config": "config",
    "utils.parallelism": "parallel.dims",
    "rollout.rollout_base": "rollout.base",
    "policy.model.base": "models.base",
    "policy.model": "models",
    "dispatcher.data.packer.multi_turn": "data.multi_turn",
    "policy.lora.plugin": "policy.lora",
    "policy.model.deepseek_v3": "models.deepseek_v3",
    "policy.model.qwen3_moe": "models.qwen3_moe",
    "policy.model.gpt": "models.gpt",
    "utils.ulysses": "parallel.context_parallel",
    "utils.trace": "utils.trace",
    "dispatcher.algo.base": "dispatcher.algo.grpo",
    "utils.distributed": "utils.dist_util",
    "utils.tools_use.hermes_tool_parser": "utils.tools_use",
    "utils.tools_use.schema": "utils.tools_use",
    "utils.tools_use.base_tool": "utils.tools_use",
    "utils.tools_use.base_tool_parser": "utils.tools_use",
    "utils.tools_use.tool_agent": "utils.tools_use",
    "rollout.schema": "rollout.base",
    "utils.model_config": "utils.extension",
    "policy.trainer.llm_trainer": "policy.trainer",
    "policy.trainer.llm_trainer.grpo_trainer": "policy.trainer.grpo_trainer",
    "policy.trainer.llm_trainer.sft_trainer": "policy.trainer.sft_trainer",
    "policy.trainer.llm_trainer.dpo_trainer": "policy.trainer.dpo_trainer",
    "policy.trainer.llm_trainer.llm_trainer": "policy.trainer.llm_trainer",
    "dispatcher.data.packer.tensor_data_packer": "data.packer",
    "dispatcher.data.packer.trajectory_packer": "data.packer",
    "dispatcher.data.packer.hf_vlm_data_packer": "data.packer",
}


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name):
        self.real_name = real_name

    def create_module(self, spec):
        return importlib.import_module(self.real_name)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        rest = fullname[len(__name__) + 1:]
        real = _TARGET + "." + _MOVED.get(rest, rest)
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real))
        locations = getattr(importlib.import_module(real), "__path__", None)
        if locations is None and any(k.startswith(rest + ".") for k in _MOVED):
            locations = []          # a plain module here, a package in the reference: its moved children resolve too
        spec.submodule_search_locations = locations
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
