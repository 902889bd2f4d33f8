"""Controller -> replica commands.

A command is a flat dict (class fields) packed with msgpack and published on the target replica's command
stream; scope LOCAL commands concern one replica, GLOBAL ones are sent to every replica they name. Field
names follow cosmos_rl/dispatcher/command.py:27-662 so that either side can be swapped.
"""
from __future__ import annotations

import uuid
from typing import Any, Callable, Dict, List, Optional, Type

import msgpack


class CommandType:
    WEIGHT_RESUME = "WEIGHT_RESUME"
    BUILD_MESH = "BUILD_MESH"
    POLICY_TO_POLICY_BROADCAST = "POLICY_TO_POLICY_BROADCAST"
    POLICY_TO_POLICY_UNICAST = "POLICY_TO_POLICY_UNICAST"
    POLICY_TO_ROLLOUT_UNICAST = "POLICY_TO_ROLLOUT_UNICAST"
    ROLLOUT_TO_ROLLOUT_BROADCAST = "ROLLOUT_TO_ROLLOUT_BROADCAST"
    STOP = "STOP"
    DATA_FETCH = "DATA_FETCH"
    TRAINING_COMPLETE = "TRAINING_COMPLETE"
    DUMMY = "DUMMY"


class CommandScope:
    GLOBAL = 0
    LOCAL = 1


_REGISTRY: Dict[str, Type["Command"]] = {}


class Command:
    command_type: str = CommandType.DUMMY
    scope_default: int = CommandScope.LOCAL

    def __init__(self, uuid_value: Optional[str] = None, scope: Optional[int] = None, **_ignored):
        self.uuid_value = uuid_value or str(uuid.uuid4())
        self.scope = self.scope_default if scope is None else scope
        self.command_type = type(self).command_type

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        _REGISTRY[cls.command_type] = cls

    # ------------------------------------------------------------------ wire format
    def to_dict(self) -> Dict[str, Any]:
        return dict(self.__dict__)

    def pack(self) -> bytes:
        return msgpack.packb(self.to_dict(), use_bin_type=True)

    @staticmethod
    def depack(data: bytes) -> "Command":
        d = msgpack.unpackb(data, raw=False, strict_map_key=False)
        return Command.from_dict(d)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "Command":
        cls = _REGISTRY.get(d.get("command_type"))
        if cls is None:
            raise ValueError(f"unknown command type {d.get('command_type')!r}")
        obj = cls.__new__(cls)
        obj.__dict__.update(d)
        return obj

    def __repr__(self):
        body = ", ".join(f"{k}={v!r}" for k, v in self.__dict__.items() if k not in ("uuid_value",))
        return f"{type(self).__name__}({body})"


class WeightResumeCommand(Command):
    """First policy replica: load weights (checkpoint if resuming, else the HF model)."""
    command_type = CommandType.WEIGHT_RESUME

    def __init__(self, replica_name: str, **kw):
        super().__init__(**kw)
        self.replica_name = replica_name


class BuildMeshCommand(Command):
    """(Re)build the inter-replica communicator: replica name -> rank in the replica-level mesh."""
    command_type = CommandType.BUILD_MESH
    scope_default = CommandScope.GLOBAL

    def __init__(self, replica_name_to_rank: Dict[str, int], **kw):
        super().__init__(**kw)
        self.replica_name_to_rank = replica_name_to_rank


class PolicyToPolicyBroadcastCommand(Command):
    command_type = CommandType.POLICY_TO_POLICY_BROADCAST
    scope_default = CommandScope.GLOBAL

    def __init__(self, src_replica_name: str, dst_replica_names: List[str], total_steps: int = 0, **kw):
        super().__init__(**kw)
        self.src_replica_name = src_replica_name
        self.dst_replica_names = dst_replica_names
        self.total_steps = total_steps


class PolicyToPolicyUnicastCommand(Command):
    command_type = CommandType.POLICY_TO_POLICY_UNICAST

    def __init__(self, src_replica_name: str, dst_replica_name: str, total_steps: int = 0, **kw):
        super().__init__(**kw)
        self.src_replica_name = src_replica_name
        self.dst_replica_name = dst_replica_name
        self.total_steps = total_steps


class PolicyToRolloutUnicastCommand(Command):
    command_type = CommandType.POLICY_TO_ROLLOUT_UNICAST

    def __init__(self, src_replica_name: str, dst_replica_name: str, src_replica_size: int, dst_replica_size: int,
                 weight_step: Optional[int] = None, total_steps: Optional[int] = None,
                 do_weight_sync_check: bool = False, trainable_only: bool = False, **kw):
        super().__init__(**kw)
        self.src_replica_name = src_replica_name
        self.dst_replica_name = dst_replica_name
        self.src_replica_size = src_replica_size
        self.dst_replica_size = dst_replica_size
        self.do_weight_sync_check = do_weight_sync_check
        self.trainable_only = trainable_only
        self.weight_step = weight_step
        self.total_steps = total_steps


class RolloutToRolloutBroadcastCommand(Command):
    command_type = CommandType.ROLLOUT_TO_ROLLOUT_BROADCAST
    scope_default = CommandScope.GLOBAL

    def __init__(self, src_replica_name: str, dst_replica_names: List[str], weight_step: Optional[int] = None,
                 total_steps: Optional[int] = None, trainable_only: bool = False, **kw):
        super().__init__(**kw)
        self.src_replica_name = src_replica_name
        self.dst_replica_names = dst_replica_names
        self.weight_step = weight_step
        self.total_steps = total_steps
        self.trainable_only = trainable_only

    def replica_should_stop(self) -> bool:
        return self.weight_step is not None and self.total_steps is not None and self.weight_step >= self.total_steps


class StopCommand(Command):
    """End-of-job signal for rollout replicas; carries no collective, so it is safe at any time."""
    command_type = CommandType.STOP

    def __init__(self, replica_name: str, **kw):
        super().__init__(**kw)
        self.replica_name = replica_name


class DataFetchCommand(Command):
    """Tells a policy replica to pop ``items_count`` rollouts from its stream and train step ``global_step``."""
    command_type = CommandType.DATA_FETCH

    def __init__(self, replica_name: str, items_count: int, global_step: int, total_steps: int,
                 remain_samples_num: int = 0, do_save: bool = False, do_profile: bool = False, active_steps: int = 1,
                 rank_filter: Optional[List[int]] = None, record_shape: bool = False, profile_memory: bool = False,
                 with_stack: bool = False, with_modules: bool = False, **kw):
        super().__init__(**kw)
        self.replica_name = replica_name
        self.items_count = items_count
        self.global_step = global_step
        self.total_steps = total_steps
        self.remain_samples_num = remain_samples_num
        self.do_save = do_save
        self.do_profile = do_profile
        self.active_steps = active_steps
        self.rank_filter = rank_filter if rank_filter is not None else [0]
        self.record_shape = record_shape
        self.profile_memory = profile_memory
        self.with_stack = with_stack
        self.with_modules = with_modules

    def replica_should_stop(self) -> bool:
        return self.global_step >= self.total_steps


class TrainingCompleteCommand(Command):
    """Tells a policy replica that no further step will come (optionally: save a final checkpoint)."""
    command_type = CommandType.TRAINING_COMPLETE

    def __init__(self, replica_name: str, global_step: int, total_steps: int, final_step: Optional[int] = None,
                 checkpoint_total_steps: Optional[int] = None, remain_samples_num: int = 0, do_save: bool = False,
                 do_profile: bool = False, active_steps: int = 1, rank_filter: Optional[List[int]] = None,
                 record_shape: bool = False, profile_memory: bool = False, with_stack: bool = False,
                 with_modules: bool = False, **kw):
        super().__init__(**kw)
        self.replica_name = replica_name
        self.global_step = global_step
        self.total_steps = total_steps
        self.final_step = global_step - 1 if final_step is None else final_step
        self.checkpoint_total_steps = total_steps if checkpoint_total_steps is None else checkpoint_total_steps
        self.remain_samples_num = remain_samples_num
        self.do_save = do_save
        self.do_profile = do_profile
        self.active_steps = active_steps
        self.rank_filter = rank_filter if rank_filter is not None else [0]
        self.record_shape = record_shape
        self.profile_memory = profile_memory
        self.with_stack = with_stack
        self.with_modules = with_modules


class CommandRegistry:
    """Maps command classes to handler callables for one worker type."""

    def __init__(self):
        self._handlers: Dict[str, Callable] = {}

    def register(self, command_cls: Type[Command], handler: Callable) -> None:
        self._handlers[command_cls.command_type] = handler

    def get_command_handler(self, command_or_type) -> Optional[Callable]:
        key = command_or_type if isinstance(command_or_type, str) else command_or_type.command_type
        return self._handlers.get(key)


class PolicyCommandRegistry(CommandRegistry):
    pass


class RolloutCommandRegistry(CommandRegistry):
    pass
