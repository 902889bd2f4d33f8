"""Controller decisions and flows without any worker process: pure decision functions, registration,
prompt hand-out (version tags, throttles), staleness filter, step scheduling, weight-sync commands,
heartbeat reaping, collective-error consensus, shutdown protocol."""
import time

import pytest

from cosmos_rl_b200.comm.broker import InProcessBroker, command_stream, rollout_stream
from cosmos_rl_b200.config import Config
from cosmos_rl_b200.dispatcher import command as cmd
from cosmos_rl_b200.dispatcher.controller import Controller
from cosmos_rl_b200.dispatcher.data import SyntheticTokenDataset
from cosmos_rl_b200.dispatcher.data.schema import RLPayload
from cosmos_rl_b200.dispatcher.protocol import RegisterRequest
from cosmos_rl_b200.dispatcher.status import (compute_total_steps, need_weight_sync, rollout_is_outdated,
                                               should_broadcast_stop, should_coalesce_skip, should_save_checkpoint)
from cosmos_rl_b200.utils import constant


def test_need_weight_sync():
    kw = dict(total_steps=10, sync_weight_interval=2, validation_enabled=False, validation_freq=None)
    assert need_weight_sync(step=2, **kw) and not need_weight_sync(step=3, **kw)
    assert not need_weight_sync(step=10, **kw)          # never on the final step without validation
    kv = dict(total_steps=10, sync_weight_interval=4, validation_enabled=True, validation_freq=5)
    assert need_weight_sync(step=5, **kv) and need_weight_sync(step=10, **kv) and need_weight_sync(step=4, **kv)
    assert not need_weight_sync(step=3, **kv)


def test_should_broadcast_stop():
    base = dict(n_policy=0, had_policy_replicas=True, stop_broadcast_sent=False, validation_enabled=False,
                training_finished=True, all_rollouts_ended=False)
    assert should_broadcast_stop(**base)
    assert not should_broadcast_stop(**{**base, "had_policy_replicas": False})       # cold start
    assert not should_broadcast_stop(**{**base, "stop_broadcast_sent": True})         # one shot
    assert not should_broadcast_stop(**{**base, "validation_enabled": True})
    assert not should_broadcast_stop(**{**base, "training_finished": False})          # rescaling to zero
    assert should_broadcast_stop(**{**base, "training_finished": False, "all_rollouts_ended": True})
    assert not should_broadcast_stop(**{**base, "n_policy": 1})


def test_coalesce_and_misc_decisions():
    assert not should_coalesce_skip(coalesce_enabled=False, forced=False, last_staged_step=5, max_adopted_version=1)
    assert should_coalesce_skip(coalesce_enabled=True, forced=False, last_staged_step=5, max_adopted_version=4)
    assert not should_coalesce_skip(coalesce_enabled=True, forced=True, last_staged_step=5, max_adopted_version=4)
    assert not should_coalesce_skip(coalesce_enabled=True, forced=False, last_staged_step=-1, max_adopted_version=-1)
    assert rollout_is_outdated(consume_step=7, weight_version=1, allowed_outdated_steps=4)
    assert not rollout_is_outdated(consume_step=6, weight_version=1, allowed_outdated_steps=4)
    assert compute_total_steps(n_samples=100, n_generation=4, epochs=2, global_batch=32, max_num_steps=None) == 25
    assert compute_total_steps(n_samples=100, n_generation=4, epochs=2, global_batch=32, max_num_steps=7) == 7
    assert should_save_checkpoint(step=4, total_steps=10, enable=True, save_freq=2)
    assert should_save_checkpoint(step=10, total_steps=10, enable=True, save_freq=3)
    assert not should_save_checkpoint(step=4, total_steps=10, enable=False, save_freq=2)
    assert should_save_checkpoint(step=3, total_steps=10, enable=True, save_freq=2, force=True)


def _config(**over):
    d = {"policy": {"model_name_or_path": "tiny-qwen2", "parallelism": {"tp_size": 1, "dp_shard_size": 1}},
         "rollout": {"n_generation": 4, "batch_size": 2, "parallelism": {"tp_size": 1}},
         "train": {"train_batch_per_replica": 8, "train_policy": {"type": "grpo", "allowed_outdated_steps": 1}}}
    for k, v in over.items():
        cur = d
        parts = k.split(".")
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        cur[parts[-1]] = v
    return Config.from_dict(d)


def _reg(c, name, role, world=1, rank=0):
    c.register(RegisterRequest(replica_name=name, role=role, mesh_names=["pp", "dp_shard", "cp", "tp"],
                               ranks=[0, rank, 0, 0], group_size=[1, world, 1, 1], global_rank=rank))


def _commands(c, name, after=0):
    return [cmd.Command.depack(d) for _, d in c.broker.read(command_stream(name), after, 100, 0)]


def _payload(idx, version, n=4, tok=3):
    return RLPayload(prompt=[1, 2, 3], prompt_idx=idx, weight_version=version, completions=[[7] * tok] * n,
                     rewards=[float(i) for i in range(n)], advantages=[float(i) - 1.5 for i in range(n)],
                     completion_token_ids=[[[7]] * tok] * n)


def test_registration_commands_and_first_sync():
    c = Controller(_config(), dataset=SyntheticTokenDataset(16, 8, 100))
    assert c.policy_status_manager.total_steps == 16 * 4 // 8
    _reg(c, "r0", "ROLLOUT")
    assert _commands(c, "r0")[0].command_type == cmd.CommandType.BUILD_MESH
    _reg(c, "p0", "POLICY")
    types = [x.command_type for x in _commands(c, "p0")]
    assert types[0] == cmd.CommandType.WEIGHT_RESUME
    assert cmd.CommandType.POLICY_TO_ROLLOUT_UNICAST in types and cmd.CommandType.BUILD_MESH in types
    rtypes = [x.command_type for x in _commands(c, "r0")]
    assert cmd.CommandType.POLICY_TO_ROLLOUT_UNICAST in rtypes
    assert rtypes[-1] == cmd.CommandType.ROLLOUT_TO_ROLLOUT_BROADCAST


def test_multi_atom_replica_waits_for_all_ranks():
    c = Controller(_config(**{"policy.parallelism.dp_shard_size": 2}), dataset=SyntheticTokenDataset(16, 8, 100))
    _reg(c, "p0", "POLICY", world=2, rank=0)
    assert not _commands(c, "p0")
    _reg(c, "p0", "POLICY", world=2, rank=1)
    assert _commands(c, "p0")[0].command_type == cmd.CommandType.WEIGHT_RESUME


def test_prompt_versions_and_throttle():
    c = Controller(_config(), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    # global batch 8 rollouts = 2 prompts per step; allowed_outdated_steps=1 -> at most 2 batches in flight
    got, is_end = c.get_batched_prompt(100)
    assert len(got) == 4 and not is_end
    assert [p.weight_version for _, p in got] == [0, 0, 1, 1]
    more, _ = c.get_batched_prompt(4)
    assert more == []                                       # throttled until training consumes a batch
    assert c.policy_status_manager.samples_on_the_fly == 16


def test_step_flow_ack_sync_and_finish():
    cfg = _config()
    c = Controller(cfg, dataset=SyntheticTokenDataset(4, 8, 100))   # 4 prompts * 4 / 8 = 2 steps
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    pm = c.policy_status_manager
    assert pm.total_steps == 2
    batch, _ = c.get_batched_prompt(2)
    n_before = len(_commands(c, "p0"))
    c.put_rollouts("r0", [_payload(i, 0) for i, _ in batch], is_end=False)
    cmds = _commands(c, "p0")[n_before:]
    assert [x.command_type for x in cmds] == [cmd.CommandType.DATA_FETCH]
    assert cmds[0].global_step == 1 and cmds[0].items_count == 8
    assert len(c.broker.read(rollout_stream("p0"), 0, 100, 0)) == 8
    assert pm.current_step == 1
    # second batch arrives while step 1 is still training: buffered, not dispatched
    batch2, is_end = c.get_batched_prompt(2)
    assert is_end
    c.put_rollouts("r0", [_payload(i, 0) for i, _ in batch2], is_end=False)
    assert pm.current_step == 1 and len(pm.rollout_buffer) == 8
    n_r = len(_commands(c, "r0"))
    c.train_ack("p0", 1, 2, False, {"train/loss_avg": 0.5, "train/grad_norm": 1.0})
    # ack of step 1: weight sync (not the last step) and step 2 dispatched
    new_r = _commands(c, "r0")[n_r:]
    assert [x.command_type for x in new_r] == [cmd.CommandType.POLICY_TO_ROLLOUT_UNICAST,
                                               cmd.CommandType.ROLLOUT_TO_ROLLOUT_BROADCAST]
    assert new_r[0].weight_step == 1 and new_r[0].trainable_only
    assert pm.current_step == 2
    n_r = len(_commands(c, "r0"))
    c.train_ack("p0", 2, 2, False, {"train/loss_avg": 0.4})
    assert _commands(c, "r0")[n_r:] == []                   # no sync after the final step
    assert pm.training_finished()
    assert c.get_batched_prompt(1) == ([], True)
    # policies leave -> STOP goes to the rollouts exactly once
    c.unregister("p0")
    stops = [x for x in _commands(c, "r0") if x.command_type == cmd.CommandType.STOP]
    assert len(stops) == 1
    c.unregister("r0")
    assert c.finalized.is_set()


def test_outdated_rollouts_are_dropped_and_release_the_throttle():
    c = Controller(_config(), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    pm = c.policy_status_manager
    pm.current_step = 5
    c.get_batched_prompt(2)
    before = pm.samples_on_the_fly
    c.put_rollouts("r0", [_payload(0, 0), _payload(1, 5)], is_end=False)
    assert pm.filtered_outdated == 4 and len(pm.rollout_buffer) == 4
    assert pm.samples_on_the_fly == before - 4


def test_invalid_groups_are_discarded():
    c = Controller(_config(), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    c.get_batched_prompt(1)
    p = _payload(0, 0)
    p.valid = False
    c.put_rollouts("r0", [p], is_end=False)
    assert c.stat_invalid == 1 and not c.policy_status_manager.rollout_buffer
    assert c.policy_status_manager.samples_on_the_fly == 0


def test_heartbeat_reaping_and_mesh_rebuild(monkeypatch):
    c = Controller(_config(**{"policy.parallelism.n_init_replicas": 2}), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "p1", "POLICY")
    types0 = [x.command_type for x in _commands(c, "p0")]
    assert cmd.CommandType.BUILD_MESH in types0 and cmd.CommandType.POLICY_TO_POLICY_BROADCAST in types0
    assert c.policy_status_manager.global_batch == 16
    now = time.time()
    c.policy_status_manager.replicas["p0"].last_heartbeat = now
    c.policy_status_manager.replicas["p1"].last_heartbeat = now - constant.COSMOS_HEARTBEAT_TIMEOUT - 1
    n0 = len(_commands(c, "p0"))
    assert c.monitor_once(now) == ["p1"]
    rebuilt = _commands(c, "p0")[n0:]
    assert rebuilt and rebuilt[0].command_type == cmd.CommandType.BUILD_MESH
    assert rebuilt[0].replica_name_to_rank == {"p0": 0}
    assert c.policy_status_manager.global_batch == 8


def test_elastic_scale_up_unicasts_state():
    c = Controller(_config(), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "p1", "POLICY")
    t1 = [x.command_type for x in _commands(c, "p1")]
    assert t1 == [cmd.CommandType.BUILD_MESH, cmd.CommandType.POLICY_TO_POLICY_UNICAST]
    u = [x for x in _commands(c, "p0") if x.command_type == cmd.CommandType.POLICY_TO_POLICY_UNICAST][0]
    assert u.src_replica_name == "p0" and u.dst_replica_name == "p1"


def test_collective_error_consensus_drops_silent_replica():
    c = Controller(_config(**{"policy.parallelism.n_init_replicas": 3}), dataset=SyntheticTokenDataset(64, 8, 100))
    for n in ("p0", "p1", "p2"):
        _reg(c, n, "POLICY")
    t0 = time.time()
    c.set_replica_ncclerror("p0", "timeout", now=t0)
    c.set_replica_ncclerror("p2", "timeout", now=t0 + 1)
    assert c._settle_nccl_errors(now=t0 + 2) == []          # grace period still running
    hung = c._settle_nccl_errors(now=t0 + constant.COSMOS_NCCL_ERROR_CLEAN_REPLICA_DELAY + 1)
    assert hung == ["p1"] and "p1" not in c.policy_status_manager.replicas
    last = _commands(c, "p0")[-1]
    assert last.command_type == cmd.CommandType.BUILD_MESH and set(last.replica_name_to_rank) == {"p0", "p2"}


def test_handshake_kv_and_resume_position():
    c = Controller(_config(), dataset=SyntheticTokenDataset(10, 8, 100))
    c.kv_put("pair", "abc")
    assert c.kv_get("pair") == "abc" and c.kv_all() == {"pair": "abc"}
    c.kv_clear("pair")
    assert c.kv_get("pair") is None
    c.set_resume_info({"step": 3, "remain_samples_num": 4})
    assert c.policy_status_manager.current_step == 3 and c.data_fetcher.remain_samples_num == 4


def test_command_roundtrip_and_unknown_type():
    c = cmd.PolicyToRolloutUnicastCommand("a", "b", 4, 2, weight_step=3, total_steps=9, trainable_only=True)
    d = cmd.Command.depack(c.pack())
    assert isinstance(d, cmd.PolicyToRolloutUnicastCommand) and d.__dict__ == c.__dict__
    assert cmd.RolloutToRolloutBroadcastCommand("a", ["a"], weight_step=9, total_steps=9).replica_should_stop()
    with pytest.raises(ValueError):
        cmd.Command.from_dict({"command_type": "NOPE"})


def test_broker_blocking_read_and_groups():
    import threading
    b = InProcessBroker()
    got = []
    t = threading.Thread(target=lambda: got.extend(b.read("s", 0, 10, 2000)))
    t.start()
    time.sleep(0.05)
    b.publish("s", b"x")
    t.join(3)
    assert got == [(1, b"x")]
    b.publish("q", b"1")
    b.publish("q", b"2")
    assert b.read_group("q", "g", 1, 0) == [(1, b"1")] and b.read_group("q", "g", 5, 0) == [(2, b"2")]
    assert b.read_group("q", "g", 5, 0) == []


def test_cosmos_cli_against_a_live_controller(tmp_path, capsys):
    """`cosmos-cli` subcommands over HTTP against a controller served in this process."""
    import json
    import socket
    import threading
    import time

    import uvicorn

    from cosmos_rl_b200.cli import cli
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.controller import Controller
    from cosmos_rl_b200.dispatcher.data import SyntheticTokenDataset
    from cosmos_rl_b200.dispatcher.protocol import RegisterRequest, Role
    from cosmos_rl_b200.dispatcher.run_web_panel import create_app
    cfg = Config.from_dict({"policy": {"model_name_or_path": "tiny-qwen2", "parallelism": {"tp_size": 1}},
                            "rollout": {"parallelism": {"tp_size": 1}},
                            "train": {"output_dir": str(tmp_path), "train_policy": {"type": "grpo"}}})
    ctl = Controller(cfg, dataset=SyntheticTokenDataset(8, 4, 100))
    ctl.register(RegisterRequest(replica_name="policy-a", role=Role.POLICY, mesh_names=["pp", "dp_shard", "cp", "tp"],
                                 ranks=[0, 0, 0, 0], group_size=[1, 1, 1, 1], global_rank=0))
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(create_app(ctl), log_level="warning"))
    th = threading.Thread(target=server.run, kwargs={"sockets": [sock]}, daemon=True)
    th.start()
    url = f"127.0.0.1:{port}"
    for _ in range(100):
        try:
            if cli.main(["--url", url, "status"]) == 0:
                break
        except Exception:
            time.sleep(0.1)
    capsys.readouterr()
    assert cli.main(["--url", url, "replica", "ls"]) == 0
    assert "policy-a" in capsys.readouterr().out
    assert cli.main(["--url", url, "replica", "lsr", "policy-a"]) == 0
    assert json.loads(capsys.readouterr().out)["name"] == "policy-a"
    assert cli.main(["--url", url, "replica", "lsr", "nobody"]) == 1
    capsys.readouterr()
    assert cli.main(["--url", url, "algo", "config"]) == 0
    assert json.loads(capsys.readouterr().out)["policy"]["model_name_or_path"] == "tiny-qwen2"
    assert cli.main(["--url", url, "profile", "set", "policy-a", "--active-steps", "2"]) == 0
    assert cli.main(["--url", url, "nccl", "ls"]) == 0
    server.should_exit = True
    th.join(timeout=10)


def test_dropped_groups_are_replaced_by_fresh_prompts():
    """Dynamic sampling: a group without reward signal does not consume the job's prompt budget."""
    cfg = _config(**{"train.train_policy.variant": "dapo"})
    c = Controller(cfg, dataset=SyntheticTokenDataset(16, 8, 100))
    c.policy_status_manager.total_steps = 2                       # 2 steps * 8 rollouts / 4 per prompt = 4 prompts
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    batch, is_end = c.get_batched_prompt(4)
    assert len(batch) == 4 and not is_end                          # dapo: the stream stays open for replacements
    assert c.get_batched_prompt(4)[0] == []
    bad = _payload(batch[0][0], 0)
    bad.valid = False
    c.put_rollouts("r0", [bad], is_end=False)
    again, _ = c.get_batched_prompt(4)
    assert len(again) == 1 and again[0][1].weight_version == batch[3][1].weight_version


def test_job_that_lost_every_rollout_replica_is_ended_in_order(monkeypatch):
    """The only rollout replica stops sending heartbeats and is reaped: the policy would wait for data forever. After the
    grace period the controller sends ``TrainingComplete`` to the policy and records why; a rollout replica that
    registers in time resets the clock instead."""
    monkeypatch.setattr(constant, "COSMOS_NO_ROLLOUT_GRACE_S", 30.0)
    c = Controller(_config(), dataset=SyntheticTokenDataset(64, 8, 100))
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    now = time.time()
    c.policy_status_manager.replicas["p0"].last_heartbeat = now + 1000
    c.rollout_status_manager.replicas["r0"].last_heartbeat = now - constant.COSMOS_HEARTBEAT_TIMEOUT - 1
    assert c.monitor_once(now) == ["r0"] and c.failed is None           # reaped; the clock starts
    assert c._starved_since == now
    c.monitor_once(now + 10)
    assert c.failed is None
    _reg(c, "r1", "ROLLOUT")                                              # a replacement arrives in time
    c.rollout_status_manager.replicas["r1"].last_heartbeat = now + 1000
    c.monitor_once(now + 20)
    assert c._starved_since is None and c.failed is None
    c.rollout_status_manager.replicas["r1"].last_heartbeat = now - constant.COSMOS_HEARTBEAT_TIMEOUT - 1
    assert c.monitor_once(now + 40) == ["r1"]
    c.monitor_once(now + 60)
    assert c.failed is None                                               # 20 s into the new period
    n0 = len(_commands(c, "p0"))
    c.monitor_once(now + 75)
    assert c.failed and "no rollout replica" in c.failed
    last = _commands(c, "p0")[n0:]
    assert [x.command_type for x in last] == [cmd.CommandType.TRAINING_COMPLETE]
    c.monitor_once(now + 200)                                             # nothing is sent twice
    assert len(_commands(c, "p0")) == n0 + 1


def test_training_completes_when_the_rollout_side_left_and_the_buffer_runs_short():
    """The rollout replica reports the end of its prompt stream and leaves while a step is still training; some of its
    rollouts never made it into the buffer (dropped as outdated, say), so the planned number of steps cannot be reached.
    When the running step is acknowledged the policy must be told that training is over, not left waiting for data."""
    c = Controller(_config(), dataset=SyntheticTokenDataset(8, 8, 100))       # 8 prompts * 4 / 8 = 4 planned steps
    _reg(c, "p0", "POLICY")
    _reg(c, "r0", "ROLLOUT")
    pm = c.policy_status_manager
    assert pm.total_steps == 4
    batch, _ = c.get_batched_prompt(2)
    c.put_rollouts("r0", [_payload(i, 0) for i, _ in batch], is_end=False)        # step 1 is dispatched
    assert pm.current_step == 1
    more, _ = c.get_batched_prompt(1)
    c.put_rollouts("r0", [_payload(i, 0) for i, _ in more], is_end=True)          # half a step, then the stream ends
    assert len(pm.rollout_buffer) == 4 and not pm.complete_sent                   # step 1 is still running
    c.unregister("r0")                                                            # regular exit after the end report
    assert c.rollout_status_manager.all_ended()
    n0 = len(_commands(c, "p0"))
    c.train_ack("p0", 1, 4, False, {"train/loss_avg": 0.5})
    new = _commands(c, "p0")[n0:]
    assert [x.command_type for x in new] == [cmd.CommandType.TRAINING_COMPLETE] and pm.complete_sent
    assert not c._check_rollout_starvation(time.time() + 10_000)                  # an orderly end, not a starved job
    assert c.failed is None
