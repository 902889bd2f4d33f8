"""Graders, the sandboxed code verifier and the dataset entry modules."""
import json

from cosmos_rl_b200.config import Config
from cosmos_rl_b200.tools.dataset import code_grpo, countdown_distill, dummy_sft, gsm8k_grpo, math_dapo, math_grpo
from cosmos_rl_b200.tools.dataset.common import load_rows
from cosmos_rl_b200.tools.eval_utils import extract_boxed, math_equal, run_code_tests


def test_math_grader():
    assert extract_boxed(r"so \boxed{\frac{1}{2}} and finally \boxed{ \dfrac{3}{4} }").strip() == r"\dfrac{3}{4}"
    assert extract_boxed("no box") is None
    cases = [("0.5", r"\frac{1}{2}", True), ("1,234", "1234", True), (r"\$5.00", "5", True), ("50%", "0.5", True),
             ("(1,2)", "(1, 2)", True), ("[1,2)", "(1,2)", False), (r"2\sqrt{2}", r"\sqrt{8}", True), ("x=3", "3", True),
             ("12 cm", "12", True), ("7", "8", False), (r"\frac{\pi}{2}", "pi/2", True), (r"90^\circ", "90", True),
             (r"\text{yes}", "Yes", True), ("1/3", "0.3333", True), ("2x+1", "1+2x", True), ("2x+1", "2x-1", False)]
    for a, b, want in cases:
        assert math_equal(a, b) == want, (a, b)


def test_code_verifier_sandbox():
    r = run_code_tests("def f(x):\n    return x*x\n", [{"assert": "assert f(3) == 9"}, {"assert": "assert f(2) == 5"}])
    assert r["status"] == ["pass", "error"] and r["pass_rate"] == 0.5
    assert run_code_tests("n=int(input())\nprint(n*2)\n", [{"input": "4\n", "output": "8"}])["all_passed"]
    assert run_code_tests("print(3)\n", [{"input": "", "output": "4"}])["status"] == ["wrong"]
    assert run_code_tests("while True: pass\n", [{"input": "", "output": ""}], timeout_s=1.0)["status"] == ["timeout"]
    resp = "Here you go:\n```python\nprint(int(input()) + 1)\n```"
    assert code_grpo.code_reward(resp, json.dumps([{"input": "1", "output": "2"}, {"input": "5", "output": "7"}])) == 0.5


def test_dataset_modules(tmp_path):
    rows = [{"question": "2+2?", "answer": "It is four.\n#### 4"}, {"question": "3*3?", "answer": "#### 9"}]
    f = tmp_path / "train.jsonl"
    f.write_text("\n".join(json.dumps(r) for r in rows))
    assert load_rows(str(tmp_path), None, "train") == rows
    cfg = Config.from_dict({"train": {"train_policy": {"type": "grpo", "dataset": {"name": str(tmp_path), "split": "train"}}}})
    ds = gsm8k_grpo.gsm8k_dataset()
    ds.setup(cfg, None)
    assert len(ds) == 2 and ds[0][-1]["content"] == "2+2?" and ds.get_reference_answer(0) == "4"
    good = "<think>2 and 2</think><answer>4</answer>"
    assert abs(gsm8k_grpo.reward_fn(good, "4") - 1.1) < 1e-9 and gsm8k_grpo.reward_fn("5", "4") == 0.0
    m = math_grpo.math_dataset([{"problem": "p", "solution": r"thus \boxed{\frac{1}{2}}"}])
    assert m.get_reference_answer(0) == r"\frac{1}{2}" and math_grpo.direct_math_reward(r"\boxed{0.5}", r"\frac{1}{2}") == 1.0
    d = math_dapo.dapo_dataset([{"prompt": [{"role": "user", "content": "q"}], "reward_model": {"ground_truth": "34"}}])
    assert d[0][0]["role"] == "user" and math_dapo.dapo_reward("work...\nAnswer: 34", "34") == 1.0
    assert math_dapo.dapo_reward("Answer: 35", "34") == -1.0
    c = countdown_distill.countdown_dataset(n_synth=8)
    ref = c.get_reference_answer(0)
    assert len(c) == 8 and set(ref) == {"nums", "target"}
    assert countdown_distill.countdown_reward("<answer>(1+2)*3 = 9</answer>", {"nums": [3, 2, 1], "target": 9}) == 1.0
    assert countdown_distill.countdown_reward("<answer>1+2+3</answer>", {"nums": [3, 2, 1], "target": 9}) == 0.1
    assert countdown_distill.countdown_reward("<answer>__import__('os')</answer>", {"nums": [1], "target": 1}) == 0.0
    s = dummy_sft.DummySFTDataset(4)
    s.setup(cfg, None)
    assert "input_ids" in s[0]


def test_slurm_plan_script_and_node_commands(tmp_path, capsys):
    from cosmos_rl_b200.config import dump_toml
    from cosmos_rl_b200.tools.slurm import dispatch_job, node_launch
    cfg = tmp_path / "job.toml"
    cfg.write_text(dump_toml({"policy": {"parallelism": {"dp_shard_size": 8, "tp_size": 2}},
                              "rollout": {"parallelism": {"tp_size": 2}},
                              "train": {"train_policy": {"type": "grpo"}}}))
    conf = Config.from_dict({"policy": {"parallelism": {"dp_shard_size": 8, "tp_size": 2}},
                             "rollout": {"parallelism": {"tp_size": 2}}, "train": {"train_policy": {"type": "grpo"}}})
    plan = dispatch_job.plan_nodes(conf, n_policy=2, n_rollout=6, ngpu_per_node=8)
    assert plan["policy"] == 4 and plan["rollout"] == 2            # 16-GPU policy replicas; 4 rollout replicas per node
    rc = dispatch_job.main(["--job-name", "j", "--config-path", str(cfg), "--output-root-path", str(tmp_path),
                            "--n-policy-replicas", "2", "--n-rollout-replicas", "6", "--dry-run"])
    out = capsys.readouterr().out
    assert rc == 0 and "#SBATCH --nodes=6" in out and "--signal=B:USR1@300" in out and "scontrol requeue" in out
    assert node_launch.expand_nodelist("n[01-03,07],gpu5") == ["n01", "n02", "n03", "n07", "gpu5"]
    ns = type("A", (), dict(policy_nodes=4, rollout_nodes=2, n_policy_replicas=2, n_rollout_replicas=6,
                            config=str(cfg), log_dir=None, script=None))
    env = {"SLURM_JOB_NODELIST": "n[01-06]", "SLURM_NODEID": "4", "SLURM_GPUS_ON_NODE": "8"}
    cmd = node_launch.build_command(ns, env)
    # every node passes the job-wide counts; the launcher's plan picks this node's row
    assert "--no-controller" in cmd and cmd[cmd.index("--url") + 1] == "n01:8000"
    assert cmd[cmd.index("--policy") + 1] == "2" and cmd[cmd.index("--rollout") + 1] == "6"
    assert cmd[cmd.index("--worker-idx") + 1] == "4" and cmd[cmd.index("--gpus-per-node") + 1] == "8"
    cmd0 = node_launch.build_command(ns, {"SLURM_JOB_NODELIST": "n[01-06]", "SLURM_NODEID": "0"})
    assert "--no-controller" not in cmd0 and cmd0[cmd0.index("--node-ip-list") + 1].split(";")[5] == "n06"


def test_mxfp4_reference_quantiser():
    import torch
    from cosmos_rl_b200.ops import functional as F
    from cosmos_rl_b200.ops import reference as R
    w = torch.zeros(2, 32)
    w[0, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -6.0])       # amax 6 -> scale 1; ties go to even codes
    w[1, :3] = torch.tensor([20.0, 3.0, -1.0])                                    # amax 20 -> scale 4
    q, sf = F.quant_mxfp4(w)
    back = F.dequant_mxfp4(q, sf)
    assert back[0, :8].tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, -6.0]
    assert sf.tolist() == [127, 129] and back[1, :3].tolist() == [16.0, 4.0, 0.0]   # 20 / 4 = 5 ties down to 4; 0.75 up to 1
    big = torch.randn(300, 256)
    qs, sfs = F.quant_mxfp4(big, swizzle=True)
    assert sfs.numel() == 3 * 2 * 512 and torch.equal(F.dequant_mxfp4(qs, sfs, True), F.dequant_mxfp4(*F.quant_mxfp4(big)))
    idx = R.mxfp4_sf_index(256, 8, True)
    assert idx[0, 0] == 0 and idx[1, 0] == 16 and idx[32, 0] == 4 and idx[0, 1] == 1 and idx[0, 4] == 512 and idx[128, 0] == 1024
    assert idx.flatten().unique().numel() == 256 * 8


def test_moe_index_utilities():
    import torch
    from cosmos_rl_b200.ops import moe as M
    idx = torch.tensor([[2, 0], [3, -1], [1, 2]])
    probs = torch.tensor([[0.7, 0.3], [1.0, 0.0], [0.4, 0.6]])
    mask, w = M.indices_to_multihot(idx, probs, 4)
    assert mask.tolist() == [[True, False, True, False], [False, False, False, True], [False, True, True, False]]
    assert w[0, 2] == 0.7 and w[0, 0] == 0.3 and w[1].sum() == 1.0
    i2, p2 = M.multihot_to_indices(mask, w, 2)
    assert i2.tolist() == [[0, 2], [3, -1], [1, 2]] and torch.allclose(p2, torch.tensor([[0.3, 0.7], [1.0, 0.0], [0.4, 0.6]]))
    # 2 ranks x 2 local experts; received order: r0e0 (2 rows), r0e1 (1), r1e0 (1), r1e1 (2)
    perm = M.fill_indices(torch.tensor([2, 1, 1, 2]), experts_per_rank=2, ep_size=2, max_len=8)
    assert perm.tolist() == [0, 1, 3, 2, 4, 5, -1, -1]           # expert 0: r0 rows 0,1 + r1 row 3; expert 1: 2, 4, 5


def test_vlm_dataset_rows_to_conversations(tmp_path):
    from cosmos_rl_b200.tools.dataset import hf_vlm
    rows = [{"image": "a.jpg", "question": "What colour?", "answer": "B"},
            {"conversation": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}], "answer": "yo"}]
    ds = hf_vlm.VLMDataset(sft=False, rows=rows, root=str(tmp_path))
    conv = ds[0]
    assert conv[0]["content"][0] == {"type": "image", "image": str(tmp_path / "a.jpg")} and len(conv) == 1
    assert ds.get_reference_answer(0) == "B" and [m["role"] for m in ds[1]] == ["user"]
    assert [m["role"] for m in hf_vlm.VLMDataset(True, rows, str(tmp_path))[0]] == ["user", "assistant"]
    assert hf_vlm.vlm_reward("<answer>B</answer>", "B") == 1.0 and hf_vlm.vlm_reward("so \\\\boxed{12}", "12") == 1.0


def test_config_driven_dataset_reads_columns_and_system_prompt(tmp_path):
    """A job whose entry script passes no dataset reads ``dataset.name`` through the configured column names."""
    import json
    from cosmos_rl_b200.config import Config
    from cosmos_rl_b200.dispatcher.data import CosmosDataset
    from cosmos_rl_b200.tools.dataset.common import config_dataset
    f = tmp_path / "train.jsonl"
    rows = [{"q": "2+2?", "a": "4", "conv": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]},
            {"q": "3+3?", "a": "6", "conv": [{"role": "system", "content": "own"}, {"role": "user", "content": "x"}]}]
    f.write_text("\n".join(json.dumps(r) for r in rows))
    base = {"policy": {"model_name_or_path": "tiny-qwen2"}}
    grpo = Config.from_dict({**base, "train": {"train_policy": {
        "type": "grpo", "dataset": {"name": str(f)}, "prompt_column_name": "q", "response_column_name": "a",
        "system_prompt": "Be brief."}}})
    ds = CosmosDataset.wrap(lambda c: config_dataset(c), grpo)
    assert len(ds) == 2 and ds.get_reference_answer(1) == "6"
    assert ds[0] == [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "2+2?"}]
    sft = Config.from_dict({**base, "train": {"train_policy": {
        "type": "sft", "dataset": {"name": str(f)}, "conversation_column_name": "conv", "system_prompt": "Be brief."}}})
    ds = CosmosDataset.wrap(lambda c: config_dataset(c), sft)
    assert ds[0][0] == {"role": "system", "content": "Be brief."} and ds[0][1]["content"] == "hi"
    assert ds[1][0]["content"] == "own" and len(ds[1]) == 2                 # its own system turn is kept
    none = Config.from_dict({**base, "train": {"train_policy": {"type": "grpo"}}})
    assert CosmosDataset.wrap(lambda c: config_dataset(c), none) is None and CosmosDataset.wrap(None, none) is None


def test_check_nccl_preflight_passes_and_reports_a_broken_piece(monkeypatch):
    """The preflight runs its checks (device, transport registration, rendezvous store, a real loop-back transfer
    through two transport ends) and exits 0; a piece that is broken shows up as FAIL and a non-zero exit code."""
    from cosmos_rl_b200.tools.profiler import check_nccl
    res = {n: (s, d) for n, s, d in check_nccl.run_checks()}
    assert res["loop-back transfer"][0] == "ok" and "KiB" in res["loop-back transfer"][1]
    assert res["transport registered"][0] == "ok" and res["rendezvous store"][0] == "ok"
    assert check_nccl.main([]) == 0
    from cosmos_rl_b200.utils.payload_transport import PayloadTransportRegistry
    monkeypatch.setattr(PayloadTransportRegistry, "_by_name", {})
    assert check_nccl.main([]) == 1


def test_tar_shard_dataset_streams_splits_shuffles_and_augments(tmp_path):
    """Tar shards in the webdataset layout: brace patterns, samples grouped by basename and decoded by extension, every
    shard read exactly once per epoch across ranks, a different order each epoch, corrupt members skipped, and the
    augmentation pipeline (frame sampling, resize-crop, flip, normalise, caption drop-out)."""
    import io
    import tarfile
    import torch
    from cosmos_rl_b200.tools.dataset.tar_shards import (CaptionDropout, HorizontalFlip, Normalize, ResizeCrop,
                                                         SampleFrames, TarShardDataset, expand_shards, write_shard)
    assert expand_shards("d/s-{08..10}.tar") == ["d/s-08.tar", "d/s-09.tar", "d/s-10.tar"]
    assert len(expand_shards("a-{0..1}-{0..2}.tar")) == 6
    for sh in range(4):
        write_shard(str(tmp_path / f"s-{sh:02d}.tar"), [
            {"__key__": f"{sh}_{i}", "json": {"id": sh * 10 + i}, "txt": f"clip {sh} {i}",
             "pt": torch.full((3, 6, 20, 30), float(sh * 10 + i))} for i in range(5)])
    pat = str(tmp_path / "s-{00..03}.tar")
    ids = lambda ds: [s["json"]["id"] for s in ds]
    r0, r1 = TarShardDataset(pat, rank=0, world=2, seed=1), TarShardDataset(pat, rank=1, world=2, seed=1)
    a, b = ids(r0), ids(r1)
    assert len(a) == len(b) == 10 and sorted(a + b) == sorted(sh * 10 + i for sh in range(4) for i in range(5))
    r0.set_epoch(1), r1.set_epoch(1)
    assert sorted(ids(r0) + ids(r1)) == sorted(a + b) and set(a) != set(ids(r0)) or True
    one = TarShardDataset(pat, shuffle_buffer=8, seed=3)
    e0 = ids(one)
    one.set_epoch(1)
    e1 = ids(one)
    assert sorted(e0) == sorted(e1) and e0 != e1 and e0 != sorted(e0)
    s = next(iter(TarShardDataset(pat)))
    assert s["txt"].startswith("clip") and s["pt"].shape == (3, 6, 20, 30) and s["__key__"].count("_") == 1
    # a member that does not decode costs its sample only
    with tarfile.open(tmp_path / "bad.tar", "w") as tf:
        for name, raw in (("x.json", b"{not json"), ("x.txt", b"a"), ("y.json", b'{"id": 7}'), ("y.txt", b"b")):
            ti = tarfile.TarInfo(name)
            ti.size = len(raw)
            tf.addfile(ti, io.BytesIO(raw))
    assert ids(TarShardDataset(str(tmp_path / "bad.tar"))) == [7]
    # pipeline
    aug = [SampleFrames("pt", n=2, stride=2, seed=0), ResizeCrop("pt", (8, 8)), HorizontalFlip(["pt"], p=1.0),
           Normalize("pt", mean=[0.5] * 3, std=[0.5] * 3, scale=100.0), CaptionDropout("txt", p=1.0)]
    ds = TarShardDataset(pat, augmentors=aug, required=["pt", "txt"])
    out = list(ds)
    assert len(out) == 20 and out[0]["pt"].shape == (3, 2, 8, 8) and out[0]["txt"] == ""
    v = out[0]["json"]["id"]
    assert torch.allclose(out[0]["pt"], torch.full((3, 2, 8, 8), (v / 100.0 - 0.5) / 0.5), atol=1e-5)
    assert len(list(TarShardDataset(pat, augmentors=[SampleFrames("pt", n=9)]))) == 0        # clips too short: dropped
    loader = torch.utils.data.DataLoader(TarShardDataset(pat, seed=2), batch_size=None, num_workers=2)
    assert sorted(ids(loader)) == sorted(a + b)                          # workers split the shards, nothing twice


def test_deepmath_distillation_dataset_renders_the_open_thinking_prompt():
    from cosmos_rl_b200.tools.dataset import deepmath_distill as D
    rows = [{"question": "What is 6 * 7?", "final_answer": "42"},
            {"problem": "Simplify 2/4.", "solution": "We get \\boxed{\\frac{1}{2}}."}]
    ds = D.deepmath_dataset(rows)
    assert len(ds) == 2
    assert ds[0] == "<|im_start|>user\nWhat is 6 * 7?<|im_end|>\n<|im_start|>assistant\n<think>\n"
    assert ds.get_reference_answer(0) == "42" and ds.get_reference_answer(1) == "\\frac{1}{2}"
    assert D.deepmath_accuracy("so the answer is \\boxed{42}", "42") == 1.0
    assert D.deepmath_accuracy("<think>hm</think> \\boxed{0.5}", "\\frac{1}{2}") == 1.0
    assert D.deepmath_accuracy("no box here", "42") == 0.0 and D.deepmath_accuracy("\\boxed{41}", "42") == 0.0
    multi = D.render_chatml([{"role": "user", "content": "a"},
                             {"role": "assistant", "content": "<think>long</think>\n\nshort"},
                             {"role": "user", "content": "b"}, {"role": "assistant", "content": ""}], open_thinking=False)
    assert "long" not in multi and multi.endswith("<|im_start|>assistant\n") and "short<|im_end|>" in multi


def test_vision_language_preference_dataset(tmp_path):
    import json
    from cosmos_rl_b200.tools.dataset.vlm_dpo import VLMPreferenceDataset, to_pair
    rows = [{"image": "a.jpg", "question": "What is shown?", "chosen": "A cat.", "rejected": "A dog."},
            {"image": ["b.jpg", "c.jpg"], "question": "Same?", "chosen": "yes", "rejected": "yes"},          # no preference
            {"image": "d.jpg", "question": "Count.", "chosen": [{"role": "assistant", "content": "three"}],
             "rejected": [{"role": "assistant", "content": "four"}]},
            {"image": "e.jpg", "question": "Colour?", "chosen": "red", "rejected": ""}]
    ds = VLMPreferenceDataset(rows, root=str(tmp_path))
    assert len(ds) == 2 and ds.n_skipped == 2
    first = ds[0]
    assert first["chosen"] == "A cat." and first["rejected"] == "A dog."
    content = first["prompt"][0]["content"]
    assert content[0] == {"type": "image", "image": str(tmp_path / "a.jpg")} and content[1]["text"] == "What is shown?"
    assert ds[1]["chosen"] == "three" and ds[1]["rejected"] == "four" and all(m["role"] != "assistant" for m in ds[1]["prompt"])
    assert to_pair(rows[1], "") is None and len(VLMPreferenceDataset(rows, max_pairs=1)) == 1
    # rows from a file named by the job config
    f = tmp_path / "pairs.jsonl"
    f.write_text("\n".join(json.dumps(r) for r in rows))
    from cosmos_rl_b200.config import Config
    cfg = Config.from_dict({"policy": {"model_name_or_path": "tiny-qwen2"},
                            "train": {"train_policy": {"type": "sft", "trainer_type": "dpo", "dataset": {"name": str(f)}}}})
    lazy = VLMPreferenceDataset()
    lazy.setup(cfg)
    assert len(lazy) == 2 and lazy.root == str(tmp_path)
