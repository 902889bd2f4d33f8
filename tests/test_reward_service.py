"""Reward service: wire format, handlers, and the HTTP round trip (enqueue -> pending -> scores, push, errors)."""
import socket
import threading
import time

import pytest
import torch

from cosmos_rl_b200.reward_service import decode_request, encode_request
from cosmos_rl_b200.reward_service.client import RewardClient
from cosmos_rl_b200.reward_service.handler import BaseRewardHandler, RewardHandlerRegistry
from cosmos_rl_b200.reward_service.server import RewardService, build_app


def test_protocol_round_trip_and_rejects_bad_sizes():
    x = torch.randn(2, 3, 4, 8, 8).to(torch.bfloat16)
    fns, meta, y = decode_request(encode_request(["sharpness"], {"fps": 8}, x))
    assert fns == ["sharpness"] and meta == {"fps": 8} and torch.equal(x, y)
    assert decode_request(encode_request(["prompt_keyword"], {"texts": ["a"]}))[2] is None
    with pytest.raises(ValueError):
        decode_request(encode_request(["sharpness"], {}, x)[:-3])


def test_builtin_handlers():
    sharp = RewardHandlerRegistry.create("sharpness")
    flat = torch.full((1, 3, 16, 16), 0.5)
    noisy = torch.rand(1, 3, 16, 16)
    s = sharp.calculate_reward(torch.cat([flat, noisy]), {})
    assert s["scores"]["sharpness"][0] < 1e-9 < s["scores"]["sharpness"][1] and s["input_info"]["shape"] == [2, 3, 16, 16]
    smooth = RewardHandlerRegistry.create("temporal_smoothness")
    still = torch.rand(1, 3, 1, 8, 8).expand(1, 3, 4, 8, 8)
    v = smooth.score(torch.cat([still, torch.rand(1, 3, 4, 8, 8)]), {})["temporal_smoothness"]
    assert v[0] == 0.0 and v[1] < -0.05
    kw = RewardHandlerRegistry.create("prompt_keyword")
    assert kw.score(None, {"keywords": ["red", "car"], "texts": ["A red truck", "red car"]})["prompt_keyword"] == [0.5, 1.0]


def test_http_round_trip(tmp_path):
    import uvicorn

    @RewardHandlerRegistry.register("slow_mean")
    class SlowMean(BaseRewardHandler):
        def score(self, media, metadata):
            time.sleep(0.3)
            return {"slow_mean": media.float().mean(dim=tuple(range(1, media.dim()))).tolist()}

    net = torch.jit.script(torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(3 * 1 * 4 * 4, 1)))
    torch.jit.save(net, str(tmp_path / "rm.pt"))
    svc = RewardService(["sharpness", "slow_mean", "torchscript"], num_workers=2,
                        handler_options={"torchscript": {"model_path": str(tmp_path / "rm.pt")}})
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(build_app(svc), log_level="warning"))
    th = threading.Thread(target=server.run, kwargs={"sockets": [sock]}, daemon=True)
    th.start()
    cli = RewardClient(f"http://127.0.0.1:{port}", timeout_s=20)
    for _ in range(100):
        try:
            assert cli.ping()["rewards"] == ["sharpness", "slow_mean", "torchscript"]
            break
        except Exception:
            time.sleep(0.1)
    x = torch.rand(2, 3, 4, 4)
    key = cli.enqueue(["slow_mean", "sharpness", "torchscript"], {"prompt": "p"}, x)
    assert cli.pull(key, block=False) is None                       # still pending: the slow handler sleeps
    res = cli.pull(key)
    assert torch.allclose(torch.tensor(res["slow_mean"]["scores"]["slow_mean"]), x.mean(dim=(1, 2, 3)), atol=1e-6)
    want = net(x.unsqueeze(2)).flatten()
    assert torch.allclose(torch.tensor(res["torchscript"]["scores"]["model_score"]), want, atol=1e-5)
    import requests
    bad = requests.post(f"http://127.0.0.1:{port}/api/reward/enqueue", data=encode_request(["nope"], {}, x))
    assert bad.status_code == 400 and "not served" in bad.text
    requests.post(f"http://127.0.0.1:{port}/api/reward/push", json={"uuid": "ext", "reward_fn": "human", "scores": [1.0]})
    assert cli.pull("ext", ["human"])["human"]["scores"] == [1.0]
    server.should_exit = True
    th.join(timeout=10)
    svc.close()


def test_remote_reward_calculator_scores_a_group_through_the_service(monkeypatch):
    """``use_remote_reward``: the completions of a prompt go to the service as one tensor; weights, per-function and
    total clipping are applied; advantages are centred within the group."""
    import uvicorn
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data.schema import RLPayload
    from cosmos_rl_b200.reward.dispatcher import RemoteRewardCalculator, make_reward_calculator

    @RewardHandlerRegistry.register("plain_mean")
    class PlainMean(BaseRewardHandler):
        def score(self, media, metadata):
            return {"mean": media.float().mean(dim=tuple(range(1, media.dim()))).tolist()}

    svc = RewardService(["plain_mean"], num_workers=1)
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(build_app(svc), log_level="warning"))
    threading.Thread(target=server.run, kwargs={"sockets": [sock]}, daemon=True).start()
    cli = RewardClient(f"http://127.0.0.1:{port}", timeout_s=20)
    for _ in range(100):
        try:
            cli.ping()
            break
        except Exception:
            time.sleep(0.1)
    c = Config.from_dict({"train": {"train_policy": {"type": "grpo", "use_remote_reward": True, "remote_reward": {
        "scale": 2.0, "reward_clip_max": 1.5,
        "reward_fns": [{"name": "plain_mean", "weight": 1.0, "score_key": "mean", "clip_max": 0.6}]}}}})
    monkeypatch.setenv("REMOTE_REWARD_URL", f"http://127.0.0.1:{port}/api/reward/enqueue")
    calc = make_reward_calculator(c)
    assert isinstance(calc, RemoteRewardCalculator) and calc.url == f"http://127.0.0.1:{port}"
    comps = [torch.full((3, 1, 4, 4), v) for v in (0.1, 0.5, 0.9)]
    p = calc.compute(RLPayload(prompt="a cat", prompt_idx=0, completions=comps))
    assert p.rewards == pytest.approx([0.2, 1.0, 1.2])        # 0.9 clipped to 0.6 before the scale of 2
    assert abs(sum(p.advantages)) < 1e-5 and p.advantages[2] > p.advantages[0]
    server.should_exit = True
