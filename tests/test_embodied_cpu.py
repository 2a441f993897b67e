"""Embodied stack on CPU: config layers, policies, trainer (single process, DDP / ZeRO-1 / FSDP over gloo), resume,
LoRA, optimizer pieces, eval transport + decoders + orchestrator."""
import json
import math
import os

import numpy as np
import pytest
import torch

from loongforge_b200.embodied import checkpoint as ckpt
from loongforge_b200.embodied.config import EmbodiedArgs, parse_args, validate
from loongforge_b200.embodied.models import POLICY_PRESETS, build_policy
from tests.dist_utils import run_distributed

# skeleton fields for the shared skeleton, `size` for the policies with an architecture of their own (Pi0.5, GR00T)
SMALL = dict(hidden=32, layers=1, heads=2, expert_hidden=32, expert_layers=1, size="tiny")


def _args(tmp, **kw):
    base = dict(model_name="pi05", model_overrides=dict(SMALL), train_steps=4, per_device_batch_size=2, image_size=28,
                action_horizon=4, output_dir=str(tmp), log_interval=1, lr=1e-3)
    base.update(kw)
    return validate(EmbodiedArgs(**base))


def test_config_layers(tmp_path):
    y = tmp_path / "c.yaml"
    y.write_text("model_name: groot_n1_6\nlr: 0.5\nstrategy: zero1\n")
    a = parse_args(["--config", str(y), "lr=0.25", "fsdp_wrap_patterns=[a.*, b]", "bf16=true"])
    assert a.model_name == "groot_n1_6" and a.lr == 0.25 and a.strategy == "zero1"
    assert a.fsdp_wrap_patterns == ["a.*", "b"] and a.bf16 is True
    with pytest.raises(KeyError):
        parse_args(["nonsense=1"])
    with pytest.raises(ValueError):
        validate(EmbodiedArgs(strategy="hsdp"))


@pytest.mark.parametrize("name", sorted(POLICY_PRESETS))
def test_policies_loss_and_sampling(name, tmp_path):
    a = _args(tmp_path, model_name=name)
    torch.manual_seed(0)
    p = build_policy(name, a)
    from loongforge_b200.embodied.data import SyntheticEpisodes, collate
    batch = collate([SyntheticEpisodes(a)[i] for i in range(2)])
    loss = p(batch)
    loss.backward()
    assert torch.isfinite(loss)
    no_grad = [n for n, q in p.named_parameters() if q.requires_grad and q.grad is None]
    if name == "pi05":
        # the loss reads the action tokens only: what the LAST language layer computes after its attention (output
        # projection, MLP, final norm) feeds nothing and gets no gradient; its keys / values do
        assert no_grad and all(".lang_norm." in n or ".lang.1." in n for n in no_grad), no_grad
        assert not any(".qkv." in n or ".input_norm." in n for n in no_grad), no_grad
    else:
        assert not no_grad, no_grad
    act = p.predict_action(batch, steps=2)
    assert act.shape == (2, a.action_horizon, a.action_dim)


def test_trainer_learns_and_resumes(tmp_path):
    from loongforge_b200.embodied.trainer import build_trainer

    a = _args(tmp_path, train_steps=6, save_interval=3, gradient_accumulation_steps=2, warmup_steps=2,
              activation_checkpoint_patterns=["policy.decoder.lang.*"])
    t = build_trainer(a)
    t.train()
    lines = [json.loads(x) for x in open(os.path.join(tmp_path, "metrics.jsonl"))]
    assert len(lines) == 6 and lines[-1]["loss"] < lines[0]["loss"] * 1.5
    assert ckpt.latest_step(str(tmp_path)) == 6
    a2 = _args(tmp_path, train_steps=8, resume=True)
    t2 = build_trainer(a2)
    t2.train()
    assert t2.step == 8 and t2.scheduler.step_count == 8


def _open_gates(model):
    """A freshly initialised Pi0.5 gates every action-expert sub-layer with zero (adaptive norms start at zero), so nothing
    inside them receives a gradient until the gates move; pretrained weights have them open. Open them as a checkpoint would."""
    torch.manual_seed(11)
    with torch.no_grad():
        for m in model.modules():
            if getattr(m, "dense", None) is not None and hasattr(m, "eps"):
                m.dense.weight.normal_(std=0.05)
                m.dense.bias.normal_(std=0.5)


def test_lora_freezes_base_and_trains_adapters(tmp_path):
    from loongforge_b200.embodied.trainer import build_trainer

    a = _args(tmp_path, lora_rank=2, lora_targets=["qkv", "o"], train_steps=2, weight_decay=0.0)
    t = build_trainer(a)
    t._setup()
    _open_gates(t.model)
    before = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    t._training_loop()
    changed = [n for n, p in t.model.named_parameters() if not torch.equal(p, before[n])]
    assert changed and all("lora_" in n for n in changed)       # no weight decay: these moved by their gradients
    assert any(".expert." in n and ".lora_b." in n for n in changed)
    assert t.lora_meta["modules"]


def test_optimizer_pieces():
    from loongforge_b200.embodied.optimizer import FP32MasterAdapter, LRScheduler, build_param_groups, clip_gradients

    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4)).to(torch.bfloat16)
    groups = build_param_groups(m, 0.1, 1e-2)
    assert sorted(g["weight_decay"] for g in groups) == [0.0, 0.1]
    opt = FP32MasterAdapter(groups, torch.optim.AdamW, lr=1e-4)
    w0 = m[0].weight.detach().clone()
    for _ in range(20):  # updates far below bf16 resolution still accumulate in the fp32 masters
        m[0].weight.grad = torch.ones_like(m[0].weight)
        opt.step()
    assert not torch.equal(m[0].weight, w0)
    s = LRScheduler(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0), "wsd", 1.0, 0.0, 2, 12)
    lrs = [s.lr_at(i) for i in range(12)]
    assert lrs[0] == 0.5 and lrs[5] == 1.0 and s.lr_at(12) < 1e-9 and 0.4 < s.lr_at(11.5) < 0.6
    p = torch.nn.Parameter(torch.zeros(3))
    p.grad = torch.tensor([3.0, float("nan"), 4.0])
    assert abs(clip_gradients([p], 1.0) - 5.0) < 1e-5 and torch.allclose(p.grad.norm(), torch.tensor(1.0), atol=1e-4)


def _dist_train(rank, world, strategy, out):
    from loongforge_b200.embodied.distributed import DistContext
    from loongforge_b200.embodied.trainer import build_trainer

    ctx = DistContext()
    ctx.rank, ctx.world, ctx.local_rank = rank, world, rank
    auto = strategy == "fsdp-auto"
    strategy = "fsdp" if auto else strategy
    a = _args(out, strategy=strategy, train_steps=3,
              fsdp_wrap_patterns=["auto"] if auto else ["backbone.blocks.*", "head.blocks.*"], fsdp_min_num_params=20000,
              fsdp_reshard_module_overrides={"*expert*": False}, fsdp_reduce_dtype="fp32" if auto else None,
              checkpoint_format="dcp" if strategy == "fsdp" else "pt", save_interval=3)
    t = build_trainer(a, ctx)
    m = t.train()
    full = sum(float(p.full_tensor().float().sum()) if hasattr(p, "full_tensor") else float(p.float().sum())
               for p in t.model.parameters())
    return m["loss"], full


@pytest.mark.parametrize("strategy", ["ddp", "zero1", "fsdp", "fsdp-auto"])
def test_distributed_strategies_agree_across_ranks(strategy, tmp_path):
    res = run_distributed(_dist_train, 2, strategy, str(tmp_path))
    assert abs(res[0][1] - res[1][1]) < 1e-3 * max(1.0, abs(res[0][1]))  # replicas hold identical weights
    assert ckpt.latest_step(str(tmp_path)) == 3


def test_msgpack_rpc_and_decoders():
    from loongforge_b200.embodied.eval import action_decoders as AD
    from loongforge_b200.embodied.eval import msgpack_numpy as mp
    from loongforge_b200.embodied.eval.transport import RPCClient, RPCError, RPCServer

    obj = {"a": np.arange(6, dtype=np.int16).reshape(2, 3), "b": [1.5, "x"], "c": {"d": np.float32(2.0)}}
    back = mp.unpackb(mp.packb(obj))
    assert back["a"].dtype == np.int16 and np.array_equal(back["a"], obj["a"]) and back["c"]["d"] == 2.0
    srv = RPCServer().start()
    srv.register("add", lambda x, y: x + y)
    cli = RPCClient(srv.host, srv.port)
    assert cli.call("ping") == "pong" and np.array_equal(cli.call("add", x=np.ones(3), y=np.ones(3)), 2 * np.ones(3))
    with pytest.raises(RPCError):
        cli.call("add", x=1)
    cli.close()
    srv.stop()
    rng = np.random.default_rng(0)
    R = AD.rot6d_to_matrix(rng.standard_normal((5, 6)))
    assert np.allclose(R @ R.transpose(0, 2, 1), np.eye(3), atol=1e-6) and np.allclose(np.linalg.det(R), 1, atol=1e-6)
    assert np.allclose(AD.rot6d_to_matrix(AD.matrix_to_rot6d(R)), R, atol=1e-6)
    assert np.allclose(AD.quat_to_matrix(AD.matrix_to_quat(R)), R, atol=1e-5)
    assert np.allclose(AD.euler_to_matrix(np.array([0.0, 0.0, np.pi / 2])) @ np.array([1.0, 0, 0]), [0, 1, 0], atol=1e-6)
    acts = np.zeros((3, 10), np.float32)
    acts[:, 0] = 0.1
    acts[:, 3:9] = AD.matrix_to_rot6d(np.eye(3))
    acts[:, 9] = [0.2, 0.7, 0.9]
    pos, rot, g = AD.decode_ee_delta(acts, np.zeros(3), np.eye(3))
    assert np.allclose(pos[:, 0], [0.1, 0.2, 0.3]) and np.allclose(rot[-1], np.eye(3)) and g.tolist() == [0, 1, 1]
    assert np.allclose(AD.decode_joint(np.ones((2, 2)), np.zeros(2), delta=True, upper=1.5), [[1, 1], [1.5, 1.5]])


def test_orchestrator_with_mock_and_real_policy(tmp_path):
    from loongforge_b200.embodied.eval.orchestrator import ENV_ADAPTERS, EvalConfig, compare_reports, run_evaluation
    from loongforge_b200.embodied.eval.policy_server import MockPolicyService, PolicyService, serve

    srv = serve(MockPolicyService(horizon=4, action_dim=3))
    goal_seeking = lambda a, obs: obs.state[3:6] + 0 * a  # noqa: E731 - adapter that jumps to the goal
    rep = run_evaluation(EvalConfig(episodes=3, port=srv.port, output_dir=str(tmp_path)), action_adapter=goal_seeking)
    srv.stop()
    assert rep["success_rate"] == 1.0 and rep["mean_steps"] == 1.0 and os.path.isfile(tmp_path / "report.json")
    a = _args(tmp_path, action_dim=3, state_dim=6)
    srv = serve(PolicyService(build_policy("pi05", a), a, denoise_steps=2))
    rep2 = run_evaluation(EvalConfig(episodes=1, port=srv.port, env_kwargs={"max_steps": 4}))
    srv.stop()
    assert rep2["policy"]["model"] == "pi05" and rep2["episodes"][0]["steps"] == 4
    assert "success_rate" in compare_reports(rep, rep2)
    with pytest.raises(RuntimeError, match="unavailable on this box"):
        ENV_ADAPTERS["libero"]()


def test_pi05_cached_sampling_and_checkpoint_names():
    """Pi0.5: the expert-only pass over cached prefix keys / values gives the velocity of the joint pass; the
    public-checkpoint name map round-trips every tensor (fused q, k, v and gate, up included)."""
    from loongforge_b200.embodied.pi05 import Pi05Config, Pi05Policy, convert_pi05_state_dict

    torch.manual_seed(0)
    c = Pi05Config.tiny()
    m = Pi05Policy(c).eval()
    B = 2
    obs = {"images": torch.randn(B, 2, 3, 28, 28), "image_masks": torch.tensor([[1, 1], [1, 0]]).bool(),
           "tokens": torch.randint(0, 512, (B, 12)), "token_mask": torch.arange(12)[None, :] < torch.tensor([[12], [7]])}
    noise, t = torch.randn(B, 6, 7), torch.full((B,), 0.7)
    with torch.no_grad():
        prefix, valid = m.embed_prefix(obs)
        suffix, cond = m.embed_suffix(noise, t)
        mask, pos = m._masks(valid, 6)
        P = valid.shape[1]
        _, joint, _ = m.decoder(prefix, suffix, mask, pos, cond)
        _, _, cache = m.decoder(prefix, None, mask[:, :P, :P], pos[:, :P], fill_cache=True)
        _, cached, _ = m.decoder(None, suffix, mask[:, P:], pos[:, P:], cond, cache=cache)
    assert torch.allclose(joint, cached, atol=1e-5)
    # a padded camera / padded instruction tokens do not change the result
    obs2 = dict(obs, tokens=obs["tokens"].clone())
    obs2["tokens"][1, 7:] = 3
    a1, a2 = m.predict_action(obs, steps=2, noise=noise), m.predict_action(obs2, steps=2, noise=noise)
    assert torch.allclose(a1, a2, atol=1e-5)
    sd = m.state_dict()
    pub = convert_pi05_state_dict(sd, c, to_public=True)
    assert "paligemma_with_expert.gemma_expert.model.layers.0.self_attn.q_proj.weight" in pub
    assert "paligemma_with_expert.paligemma.model.vision_tower.vision_model.encoder.layers.1.self_attn.k_proj.bias" in pub
    back = convert_pi05_state_dict({"model." + k: v for k, v in pub.items()}, c)
    assert set(back) == set(sd) and all(torch.equal(sd[k], back[k]) for k in sd)
    with pytest.raises(KeyError):
        convert_pi05_state_dict({**pub, "stray.weight": torch.zeros(1)}, c)


def test_groot_embodiment_specific_weights_and_alternating_context():
    """GR00T N1.6: another embodiment id selects other encoder / decoder weights; cross-attention blocks alternate
    between text and image tokens; the action-head name map round-trips."""
    from loongforge_b200.embodied.groot import GrootConfig, GrootPolicy, convert_groot_state_dict

    torch.manual_seed(0)
    c = GrootConfig.tiny()
    m = GrootPolicy(c).eval()
    B = 2
    obs = {"images": torch.randn(B, 1, 3, 28, 28), "tokens": torch.randint(0, 256, (B, 9)), "state": torch.randn(B, 7),
           "embodiment_id": torch.tensor([1, 1])}
    noise = torch.randn(B, 5, 7)
    a1 = m.predict_action(obs, noise=noise)
    a2 = m.predict_action(dict(obs, embodiment_id=torch.tensor([1, 2])), noise=noise)
    assert torch.allclose(a1[0], a2[0], atol=1e-6) and not torch.allclose(a1[1], a2[1], atol=1e-4)
    # block 0 reads text only, block 2 images only: changing the instruction leaves block-2 inputs' context mask alone
    seen = []
    for i, blk in enumerate(m.action_head.model.blocks):
        blk.register_forward_hook(lambda _m, args, _o, i=i: seen.append((i, None if len(args) < 4 else args[3])))
    m.predict_action(obs, steps=1, noise=noise)
    masks = {i: mk for i, mk in seen}
    n_img = (28 // 7 // 2) ** 2
    assert masks[1] is None and masks[3] is None
    assert masks[0][:, :n_img].sum() == 0 and masks[0][:, n_img:].all()
    assert masks[2][:, :n_img].all() and masks[2][:, n_img:].sum() == 0
    sd = {k: v for k, v in m.state_dict().items() if k.startswith("action_head.")}
    pub = convert_groot_state_dict(sd, c, to_public=True, head_only=False)
    assert "action_head.model.transformer_blocks.3.attn1.to_out.0.weight" in pub
    back = convert_groot_state_dict({**pub, "backbone.anything": torch.zeros(1)}, c)
    assert set(back) == set(sd) and all(torch.equal(sd[k], back[k]) for k in sd)


def test_eval_command_line_serves_a_trained_checkpoint_and_runs_episodes(tmp_path, capsys):
    """``python -m loongforge_b200.embodied.eval``: serve the newest checkpoint of a run, evaluate against a server."""
    from loongforge_b200.embodied.eval import __main__ as cli
    from loongforge_b200.embodied.eval.policy_server import MockPolicyService, serve
    from loongforge_b200.embodied.trainer import build_trainer

    a = _args(tmp_path, train_steps=2, save_interval=2, action_dim=3, state_dim=6, model_name="groot_n1_6")
    build_trainer(a).train()
    over = ["model_name=groot_n1_6", "model_overrides={size: tiny}", "action_dim=3", "state_dim=6", "image_size=28",
            "action_horizon=4"]
    assert cli.main(["serve", "--checkpoint", str(tmp_path), "--once"] + over) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["model"] == "groot_n1_6"
    with pytest.raises(FileNotFoundError):
        cli.main(["serve", "--checkpoint", str(tmp_path / "none"), "--once"] + over)
    srv = serve(MockPolicyService(horizon=4, action_dim=3))
    try:
        assert cli.main(["run", "--port", str(srv.port), "--episodes", "2", "--max-steps", "3",
                         "--output-dir", str(tmp_path / "ev")]) == 0
    finally:
        srv.stop()
    rep = json.load(open(tmp_path / "ev" / "report.json"))
    assert len(rep["episodes"]) == 2


def test_xvla_domains_action_spaces_and_sampler():
    """X-VLA: another domain id selects other encoder / decoder matrices and soft prompts; gripper channels are logits
    (zeroed in the inputs, sigmoid in the sampler's output); a padded view contributes nothing."""
    from loongforge_b200.embodied.xvla import EE6DSpace, XVLAConfig, XVLAPolicy

    torch.manual_seed(0)
    c = XVLAConfig.tiny(action_space="ee6d", action_dim=20, max_action_dim=20)
    m = XVLAPolicy(c).eval()
    B = 2
    obs = {"images": torch.randn(B, 2, 3, 32, 32), "tokens": torch.randint(0, 100, (B, 9)), "state": torch.randn(B, 20),
           "domain_id": torch.tensor([1, 1])}
    noise = torch.randn(B, 4, 20)
    a1 = m.predict_action(obs, steps=2, noise=noise)
    a2 = m.predict_action(dict(obs, domain_id=torch.tensor([1, 2])), steps=2, noise=noise)
    assert torch.allclose(a1[0], a2[0], atol=1e-6) and not torch.allclose(a1[1], a2[1], atol=1e-4)
    assert ((a1[..., [9, 19]] >= 0) & (a1[..., [9, 19]] <= 1)).all()  # gripper probabilities
    # the second view masked out == the second view replaced by anything
    masked = dict(obs, image_masks=torch.tensor([[1, 0], [1, 0]]).bool())
    other = dict(masked, images=torch.cat([obs["images"][:, :1], torch.randn(B, 1, 3, 32, 32)], 1))
    assert torch.allclose(m.predict_action(masked, steps=1, noise=noise), m.predict_action(other, steps=1, noise=noise), atol=1e-6)
    sp = EE6DSpace()
    pred, tgt = torch.zeros(2, 3, 20), torch.zeros(2, 3, 20)
    tgt[..., 0] = 0.1
    l = sp.compute_loss(pred, tgt)
    assert abs(float(l["regress_0"]) - 500.0 * 0.01 / 3) < 1e-5 and abs(float(l["gripper"]) - math.log(2.0)) < 1e-6
    l2 = sp.compute_loss(pred, tgt, valid=torch.tensor([True, False]))
    assert abs(float(l2["regress_0"]) - float(l["regress_0"])) < 1e-6  # padded rows leave the mean over valid rows unchanged


def _zero_worker(rank, world, tmp, steps, resume_from):
    """Identical 'reduced' gradients on every rank: the sharded optimizer must reproduce plain AdamW on all of them."""
    from loongforge_b200.embodied.optimizer import ZeroAdamW, build_param_groups

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
    names = {id(p): n for n, p in model.named_parameters()}
    opt = ZeroAdamW(build_param_groups(model, 0.1, 1e-2), names, lr=1e-2, weight_decay=0.1)
    if resume_from:
        import glob
        opt.load_local_state_dicts([torch.load(f, weights_only=False) for f in sorted(glob.glob(os.path.join(resume_from, "shard_*.pt")))])
    g = torch.Generator().manual_seed(5 + (100 if resume_from else 0))
    for _ in range(steps):
        for p in model.parameters():
            p.grad = torch.randn(p.shape, generator=g)
        opt.step()
    torch.save(opt.local_state_dict(), os.path.join(tmp, f"shard_{rank}.pt"))
    owned = sum(p.numel() for p in opt.owned())
    return [p.detach().flatten().tolist() for p in model.parameters()], owned, len(opt.state)


def test_zero_adamw_matches_adamw_and_reshards(tmp_path):
    from tests.dist_utils import run_distributed as rd

    def reference(steps_a, steps_b):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.LayerNorm(5), torch.nn.Linear(5, 3))
        from loongforge_b200.embodied.optimizer import build_param_groups
        opt = torch.optim.AdamW(build_param_groups(model, 0.1, 1e-2), lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
        for seed, n in ((5, steps_a), (105, steps_b)):
            g = torch.Generator().manual_seed(seed)
            for _ in range(n):
                for p in model.parameters():
                    p.grad = torch.randn(p.shape, generator=g)
                opt.step()
        return [p.detach().clone() for p in model.parameters()]

    d2 = tmp_path / "w2"
    d2.mkdir()
    res = rd(_zero_worker, 2, str(d2), 4, None)
    ref = reference(4, 0)
    for r in res:
        assert all(torch.allclose(torch.tensor(a), b.flatten(), atol=1e-6) for a, b in zip(r[0], ref))
    total = sum(p.numel() for p in ref)
    assert res[0][1] + res[1][1] == total and 0.3 * total < res[0][1] < 0.7 * total   # balanced partition
    assert res[0][2] + res[1][2] == len(ref)                                          # every parameter has one owner
    # the two shards resume on THREE ranks and on one
    ref2 = reference(4, 3)
    for world in (3, 1):
        dn = tmp_path / f"w{world}"
        dn.mkdir()
        res = rd(_zero_worker, world, str(dn), 3, str(d2))
        for r in res:
            assert all(torch.allclose(torch.tensor(a), b.flatten(), atol=1e-6) for a, b in zip(r[0], ref2))


def _zero_resume_worker(rank, world, out, steps, resume):
    from loongforge_b200.embodied.distributed import DistContext
    from loongforge_b200.embodied.trainer import build_trainer

    ctx = DistContext()
    ctx.rank, ctx.world, ctx.local_rank = rank, world, rank
    a = _args(out, strategy="zero1", train_steps=steps, save_interval=2, resume=resume, lr_scheduler="constant")
    t = build_trainer(a, ctx)
    t.train()
    return float(sum(p.float().sum() for p in t.model.parameters())), sorted(os.listdir(os.path.join(out, f"step_{steps:08d}")) if os.path.isdir(os.path.join(out, f"step_{steps:08d}")) else [])


def test_zero1_trainer_writes_shards_and_resumes(tmp_path):
    out = str(tmp_path)
    res = run_distributed(_zero_resume_worker, 2, out, 2, False)
    step_dir = [d for d in os.listdir(out) if d.startswith("step")][0]
    files = os.listdir(os.path.join(out, step_dir))
    assert "optim_shard_00000.pt" in files and "optim_shard_00001.pt" in files and "model_optim.pt" in files
    res2 = run_distributed(_zero_resume_worker, 2, out, 4, True)           # continues from step 2
    assert ckpt.latest_step(out) == 4 and abs(res2[0][0] - res2[1][0]) < 1e-3 * max(1.0, abs(res2[0][0]))
    assert res2[0][0] != res[0][0]


def test_fsdp_auto_planner_units():
    import torch.nn as nn
    from loongforge_b200.embodied.distributed import FSDPAutoPlanner

    class Block(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.a, self.b = nn.Linear(d, d), nn.Linear(d, d)

        def forward(self, x):
            return self.b(self.a(x))

    class Odd(nn.Module):  # parameters of two dtypes: never one unit
        def __init__(self, d):
            super().__init__()
            self.w = nn.Linear(d, d)
            self.s = nn.Linear(d, d).to(torch.bfloat16)

        def forward(self, x):
            return self.s(self.w(x).bfloat16())

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(1000, 16)                      # 16,000 parameters: a leftover leaf
            self.blocks = nn.ModuleList([Block(16) for _ in range(5)])   # 544 each
            self.odd = nn.ModuleList([Odd(16), Odd(16)])
            self.head = nn.Linear(16, 4)

    net = Net()
    p = FSDPAutoPlanner(net, min_num_params=1000, leftover_min_num_params=10000,
                        reshard_overrides={"blocks.2": 4}, reshard_default=True, reshard_root=False)
    layer_units = [u for u in p.units if u["kind"] == "layers"]
    # five blocks of 544 -> groups of two (>= 1000); the single tail block joins the last group
    assert [u["names"] for u in layer_units if u["names"][0].startswith("blocks")] == [["blocks.0", "blocks.1"], ["blocks.2", "blocks.3", "blocks.4"]]
    assert [u["reshard"] for u in layer_units if u["names"][0].startswith("blocks")] == [True, 4]
    # mixed-dtype modules are descended into: their fp32 / bf16 linears group by parent and class (272 each: below the
    # threshold even together within one parent, so they stay with the root)
    assert not any(n.startswith("odd") for u in p.units for n in u["names"])
    assert [u["names"] for u in p.units if u["kind"] == "leaf"] == [["embed"]]
    planned = sum(u["params"] for u in p.units)
    assert planned + p.root_params == sum(q.numel() for q in net.parameters())
    assert "root" in p.describe() and "blocks.0, blocks.1" in p.describe()
    q = FSDPAutoPlanner(net, min_num_params=1000, leftover_min_num_params=10000, no_wrap=["Block"])
    # blocks may not be units: the walk reaches their linears (class Linear, parent blocks.i: 2 x 272 < 1000 per parent)
    assert not any(n.startswith("blocks") for u in q.units for n in u["names"])

    class Reached(Block):
        forward = nn.Module.forward            # no forward of its own: other code calls its parts

    net2 = nn.ModuleList([Reached(16) for _ in range(4)])
    assert not FSDPAutoPlanner(net2, min_num_params=100, leftover_min_num_params=10000).units[0]["names"][0].count(".") == 0


def test_lora_selection_adapter_files_and_merge(tmp_path):
    import torch.nn as nn
    from loongforge_b200.embodied import lora as L

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.o = nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 8)

        def forward(self, x):
            return self.o(self.q(x) * self.k(x))

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Attn(), Attn()])
            self.head = nn.Linear(8, 3)

        def default_lora_targets(self):
            return ["q", "k"]

        def forward(self, x):
            for b in self.blocks:
                x = x + b(x)
            return self.head(x)

    torch.manual_seed(0)
    net, x = Net(), torch.randn(4, 8)
    y0 = net(x)
    meta = L.inject_lora(net, 2, 4.0, [], use_rslora=True, exclude=["blocks.1.k"], modules_to_save=["head"])
    assert meta["modules"] == ["blocks.0.q", "blocks.0.k", "blocks.1.q"] and meta["saved_modules"] == ["head"]
    assert net.blocks[0].q.scale == 4.0 / 2 ** 0.5
    assert torch.allclose(net(x), y0)                                        # B = 0: nothing changes yet
    train = {n for n, p in net.named_parameters() if p.requires_grad}
    assert train == {n for n in dict(net.named_parameters()) if "lora_" in n or n.startswith("head.")}
    opt = torch.optim.SGD([p for p in net.parameters() if p.requires_grad], lr=0.01)
    for _ in range(3):
        opt.zero_grad()
        net(x).pow(2).sum().backward()
        opt.step()
    y1 = net(x)
    L.save_adapter(net, str(tmp_path / "ad"), meta, {"model_name": "toy"})
    sd = torch.load(tmp_path / "ad" / L.ADAPTER_WEIGHTS)
    assert set(sd) == {n if "lora_" in n else n for n in train} and not any(".base." in k for k in sd)
    torch.manual_seed(0)
    fresh = Net()                                                            # base weights as before training
    got = L.load_adapter(fresh, str(tmp_path / "ad"))
    assert got["model_name"] == "toy" and torch.allclose(fresh(x), y1, atol=1e-6)
    assert L.merge_lora(fresh) == 3 and not any(isinstance(m, L.LoRALinear) for m in fresh.modules())
    assert torch.allclose(fresh(x), y1, atol=1e-5)
    with pytest.raises(ValueError):
        L.inject_lora(Net(), 2, 4.0, ["nothing_matches"])
    all_lin = L.inject_lora(Net(), 2, 4.0, ["all-linear"], exclude=["head"])
    assert len(all_lin["modules"]) == 6
    g = L.inject_lora(Net(), 2, 4.0, ["blocks.*.o"], dropout=0.1, init="gaussian")
    assert g["modules"] == ["blocks.0.o", "blocks.1.o"]


def test_metric_logger_and_stage_timers(tmp_path, capsys):
    import time as _t
    from loongforge_b200.embodied.logging import MetricLogger, StageTimers, flatten_config, format_block

    a = _args(tmp_path, model_overrides={"size": "tiny", "nested": {"x": 1}})
    flat = flatten_config(a)
    assert flat["model_overrides.nested.x"] == 1 and flat["model_name"] == "pi05"
    assert "model_name ..." in format_block("t", flat) and format_block("t", flat).startswith("-" * 24 + " t ")
    lg = MetricLogger(str(tmp_path), True, total_steps=30, tensorboard=True, smoothing=5, spike_factor=3.0)
    lg.log_config(a)
    stats = lg.log_param_stats(torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2)))
    assert stats["total"] == 30 and stats["trainable"] == 30
    timers = StageTimers(True)
    for step in range(1, 9):
        with timers("data"):
            _t.sleep(0.002)
        with timers("optimizer"):
            pass
        loss = 10.0 if step == 8 else 1.0
        lg.log(step, {"loss": loss, "video loss": 0.5, "lr": 1e-4}, samples=4, stage_times=timers.summary(1))
    lg.finish()
    recs = [json.loads(x) for x in open(tmp_path / "metrics.jsonl")]
    assert len(recs) == 8 and recs[-1].get("loss_spike") is True and lg.spikes == 1
    assert abs(recs[4]["loss_smoothed"] - 1.0) < 1e-9 and recs[-1]["time/data"] >= 2.0 and "eta_s" in recs[-1]
    assert recs[3]["video loss"] == 0.5
    out = capsys.readouterr().out
    assert "loss spike at step 8" in out and "time (ms) | data:" in out and "end of embodied training arguments" in out
    assert os.path.isdir(tmp_path / "tensorboard") and os.listdir(tmp_path / "tensorboard")
    assert json.load(open(tmp_path / "config.json"))["model_name"] == "pi05"
    off = StageTimers(False)
    with off("x"):
        pass
    assert off.summary() == {}


def test_transforms_normalizer_images_rotations_and_prompts(tmp_path):
    from loongforge_b200.embodied import transforms as T
    from loongforge_b200.embodied.data import hash_tokenize

    rng = np.random.default_rng(0)
    data = rng.normal(2.0, 3.0, size=(500, 4)).astype(np.float32)
    data[:, 3] = 7.0                                                    # a constant channel
    st = T.compute_stats([data[:250], data[250:]])
    assert abs(st["mean"][0] - data[:, 0].mean()) < 1e-4 and st["count"] == [500]
    for mode in ("mean_std", "min_max", "q99", "scale"):
        nz = T.Normalizer(mode, st)
        y = nz.forward(data)
        if mode in ("min_max", "q99"):
            assert y[:, :3].min() >= -1 - 1e-6 and y[:, :3].max() <= 1 + 1e-6
        inside = np.abs(y[:, :3]) < 1 if mode == "q99" else np.ones_like(y[:, :3], dtype=bool)
        back = nz.inverse(y)
        assert np.allclose(back[:, :3][inside], data[:, :3][inside], atol=1e-3), mode
    assert np.allclose(T.Normalizer("mean_std", st).forward(data)[:, 3], 7.0)            # constant channel passes through
    assert np.allclose(T.Normalizer("min_max", st).forward(data)[:, 3], 0.0)
    masked = T.Normalizer("mean_std", st, mask=[True, True, False, False]).forward(data)
    assert np.allclose(masked[:, 2], data[:, 2]) and not np.allclose(masked[:, 0], data[:, 0])
    with pytest.raises(KeyError):
        T.Normalizer("q99", {"mean": [0], "std": [1]})
    T.save_stats({"state": st}, str(tmp_path / "meta" / "stats.json"))
    assert T.load_stats(str(tmp_path))["state"]["q99"] == st["q99"]

    img = np.zeros((3, 20, 40), np.float32)
    img[:, :, 20:] = 1.0
    padded = T.resize_with_pad(img, 32, 32)
    assert padded.shape == (3, 32, 32) and padded[:, :8].max() == 0 and padded[:, 8:24, 28:].min() == 1.0
    assert T.center_crop_resize(img, 16, 16).shape == (3, 16, 16)
    aug = T.ImageAugment(seed=0)
    s = aug({"images": rng.random((2, 3, 16, 16)).astype(np.float32)})
    assert s["images"].shape == (2, 3, 16, 16) and 0 <= s["images"].min() and s["images"].max() <= 1

    eul = rng.uniform(-1, 1, size=(5, 3))
    r6 = T.RotationTransform("euler", "rot6d")
    assert r6.forward(eul).shape == (5, 6) and np.allclose(r6.inverse(r6.forward(eul)), eul, atol=1e-5)
    q = T.RotationTransform("euler", "quat")
    assert np.allclose(q.inverse(q.forward(eul)), eul, atol=1e-5)
    a, state = rng.normal(size=(4, 3)).astype(np.float32), rng.normal(size=(5,)).astype(np.float32)
    rel = T.to_relative(a, state, [True, True, False])
    assert np.allclose(rel[:, 2], a[:, 2]) and np.allclose(T.to_absolute(rel, state, [True, True, False]), a, atol=1e-6)

    p = T.Pi05Prompt(lambda t, n: hash_tokenize(t, n), 48, num_bins=256, max_state_dim=4)
    text = p.prompt("pick_up the\ncube ", np.array([-1.0, 0.0, 0.999]))
    assert text == "Task: pick up the cube, State: 0 128 255 128;\nAction: "
    assert p.prompt("x", None) == "Task: x;\nAction: "
    g = T.GrootEmbodiment({"gr1": 3})({"embodiment_tag": "gr1", "state": {"arm": [1, 2], "hand": [3]}, "actions": np.zeros((2, 2))})
    assert g["embodiment_id"] == 3
    g2 = T.GrootEmbodiment({"gr1": 3}, state_keys=["hand", "arm"])({"state": {"arm": [1, 2], "hand": [3]}, "actions": np.zeros((2, 2))})
    assert g2["embodiment_id"] == 4 and g2["state"].tolist() == [3, 1, 2]
    assert T.Cosmos3Meta.append_sentence("Pick the cube", "Robot: arm.") == "Pick the cube. Robot: arm."
    d = T.DreamZeroFlags()({"actions": np.array([[2.0, -3.0]]), "state": np.array([0.5]), "action_mask": np.zeros(1)})
    assert d["actions"].tolist() == [[1.0, -1.0]] and d["has_real_action"] == 0.0


@pytest.mark.parametrize("name", ["pi05", "dreamzero", "cosmos3"])
def test_transformed_dataset_feeds_the_trainer(name, tmp_path):
    from loongforge_b200.embodied.data import build_dataset, collate
    from loongforge_b200.embodied.trainer import build_trainer

    a = _args(tmp_path, model_name=name, model_overrides={"size": "tiny"}, use_transforms=True, image_augmentation=True,
              image_size=32, stats_samples=64, train_steps=2, video_frames=9 if name == "dreamzero" else 5 if name == "cosmos3" else 0,
              robot_description="A single-arm robot." if name == "cosmos3" else None, relative_action_mask=[True] * 7)
    ds = build_dataset(a)
    assert os.path.isfile(tmp_path / "stats.json")
    b = collate([ds[i] for i in range(2)])
    assert b["images"].shape == (2, 1, 3, 32, 32)
    assert name == "cosmos3" or b["actions"].abs().max() <= 1 + 1e-6       # q99 / min-max are bounded, mean-std is not
    if name == "dreamzero":
        assert b["has_real_action"].tolist() == [1.0, 1.0] and b["embodiment_id"].tolist() == [0, 0]
    if name == "cosmos3":
        assert b["domain_id"].tolist() == [0, 0] and b["raw_action_dim"].tolist() == [7, 7]
    nsa = ds.transform.find(__import__("loongforge_b200.embodied.transforms", fromlist=["x"]).NormalizeStateAction)
    raw = ds.base[0]
    norm = ds[0]["actions"]
    inside = (np.abs(norm) < 1) | (name == "cosmos3")           # q99 / min-max clip the tails: those do not come back
    assert inside.mean() > 0.8
    assert np.allclose(nsa.unnormalize_actions(norm, raw["state"])[inside], raw["actions"][inside], atol=1e-3)
    m = build_trainer(a).train()
    assert np.isfinite(m["loss"])


def test_policy_service_uses_training_transforms(tmp_path):
    """A server started from a run's output directory prepares observations like the training pipeline and answers in
    robot units (the statistics written during training bring the normalised prediction back)."""
    from loongforge_b200.embodied.data import build_dataset
    from loongforge_b200.embodied.eval.policy_server import PolicyService
    from loongforge_b200.embodied.eval.protocol import ActionChunk, Observation
    from loongforge_b200.embodied import transforms as T

    a = _args(tmp_path, model_name="pi05", model_overrides={"size": "tiny"}, use_transforms=True, image_size=32, stats_samples=64)
    build_dataset(a)                                            # writes stats.json
    torch.manual_seed(0)
    policy = build_policy("pi05", a)
    svc = PolicyService.from_output_dir(policy, a, denoise_steps=2)
    assert svc.transform is not None and svc.transform.find(T.Pi05Prompt) is not None
    obs = Observation({"front": np.random.default_rng(0).integers(0, 255, (48, 64, 3), dtype=np.uint8)},
                      np.linspace(-1, 1, 8).astype(np.float32), "pick up the cube")
    out = ActionChunk.from_wire(svc.predict_action(obs.to_wire()))
    assert out.actions.shape == (a.action_horizon, a.action_dim) and np.isfinite(out.actions).all()
    plain = PolicyService(policy, a, denoise_steps=2)
    nsa = svc.transform.find(T.NormalizeStateAction)
    lo, hi = np.asarray(nsa.action.s["q01"]), np.asarray(nsa.action.s["q99"])
    # the transformed service answers inside the data's action range (inverse of a [-1, 1] normalisation, up to overshoot)
    assert (out.actions > lo - 3 * (hi - lo)).all() and (out.actions < hi + 3 * (hi - lo)).all()
    assert plain.transform is None


def test_eval_metrics_resume_and_report(tmp_path):
    from loongforge_b200.embodied.eval import metrics as M
    from loongforge_b200.embodied.eval.orchestrator import EvalConfig, run_evaluation
    from loongforge_b200.embodied.eval.policy_server import MockPolicyService, serve

    lo, hi = M.wilson_interval(8, 10)
    assert abs(lo - 0.4902) < 1e-3 and abs(hi - 0.9433) < 1e-3 and M.wilson_interval(0, 0) == (0.0, 1.0)
    recs = [{"suite": "s", "task": "a", "episode": i, "seed": 0, "success": i < 3, "steps": 10 + i, "failure_reason": None if i < 3 else "timeout"}
            for i in range(4)] + [{"suite": "s", "task": "b", "episode": 0, "seed": 0, "success": False, "steps": 5, "failure_reason": "collision"}]
    tasks = M.summarize_tasks(recs)
    assert [t["task"] for t in tasks] == ["a", "b"] and tasks[0]["success_rate"] == 0.75 and tasks[0]["failure_reasons"] == {"timeout": 1}
    suite = M.summarize_suites(recs, min_episodes=2)[0]
    assert suite["episodes"] == 5 and suite["success_rate"] == 0.6 and suite["task_mean_success_rate"] == 0.75 and suite["short_tasks"] == ["b"]
    assert M.validate_episode_floor(recs, 2) == [{"suite": "s", "task": "b", "episodes": 1, "required": 2}]
    p = str(tmp_path / "r.jsonl")
    for r in recs[:2]:
        M.append_jsonl(p, r)
    with open(p, "a") as f:
        f.write('{"suite": "s", "task": "a", "epis')                      # a record cut off by an interruption
    assert len(M.load_jsonl(p)) == 2 and M.completed_keys(M.load_jsonl(p)) == {("s", "a", 0, 0), ("s", "a", 1, 0)}

    srv = serve(MockPolicyService(horizon=4, action_dim=3))
    to_goal = lambda a, obs: obs.state[3:6] + 0 * a  # noqa: E731
    out = str(tmp_path / "eval")
    cfg = EvalConfig(episodes=2, port=srv.port, output_dir=out, suite="reach", seeds=[0, 1], min_episodes=3,
                     tasks=[{"name": "easy", "env_kwargs": {"tol": 0.2}}, {"name": "never", "env_kwargs": {"tol": 0.2, "max_steps": 3}}])
    rep = run_evaluation(cfg, action_adapter=to_goal)
    assert len(M.load_jsonl(os.path.join(out, "results.jsonl"))) == 8 and rep["success_rate"] == 1.0 and len(rep["tasks"]) == 2 and rep["suites"][0]["episodes"] == 8
    assert rep["latency_ms"]["calls"] >= 8 and not rep["floor_violations"]          # 2 episodes x 2 seeds = 4 per task
    # resume: nothing runs again, one more episode per task and seed is added
    cfg.episodes = 3
    rep2 = run_evaluation(cfg, action_adapter=lambda a, obs: np.ones(3) * 5)        # the new episodes fail
    srv.stop()
    assert len(M.load_jsonl(os.path.join(out, "results.jsonl"))) == 12
    assert abs(rep2["success_rate"] - 8 / 12) < 1e-9 and len(rep2["failures"]) == 4 and rep2["failures"][0]["failure_reason"] == "timeout"
    md = open(os.path.join(out, "report.md")).read()
    assert "## Suites" in md and "| reach | easy | 6 | 4 |" in md and "## Failed episodes" in md and "## Reproduction" in md
    rows = list(__import__("csv").DictReader(open(os.path.join(out, "summary_tasks.csv"))))
    assert len(rows) == 2 and rows[0]["task"] == "easy" and float(rows[0]["ci95_high"]) <= 1.0


def test_trainer_options_pretrained_freeze_schedules_async_save(tmp_path):
    from loongforge_b200.embodied.optimizer import Lion, LRScheduler, build_optimizer
    from loongforge_b200.embodied.trainer import build_trainer, freeze_modules, load_pretrained

    a = _args(tmp_path / "a", train_steps=2, save_interval=2, async_save=True, save_training_state=False, num_workers=0,
              deterministic_mode=True, lr_scheduler="cosine_restarts", lr_num_cycles=2, lr_decay_steps=8, optimizer="lion",
              lr_mults={"policy.decoder.expert": 0.1}, profile_step_start=0, profile_step_end=1)
    t = build_trainer(a)
    t.train()
    assert isinstance(t.optimizer, Lion) and {round(g["lr_mult"], 3) for g in t.optimizer.param_groups} == {0.1, 1.0}
    assert ckpt.latest_step(str(tmp_path / "a")) == 2                       # the background writer finished and marked it
    blob = torch.load(tmp_path / "a" / "step_00000002" / "model_optim.pt", weights_only=False)
    assert blob["optim"] is None and os.listdir(tmp_path / "a" / "profile")
    sd = blob["model"]
    # a second run starts from those weights with part of the model frozen
    b = _args(tmp_path / "b", train_steps=1, pretrained_checkpoint=str(tmp_path / "a" / "step_00000002" / "model_optim.pt"),
              freeze_modules=["policy.decoder.lang.*"])
    t2 = build_trainer(b)
    t2._setup()
    got = ckpt._unwrap(t2.model).state_dict()
    assert all(torch.equal(got[k], v) for k, v in sd.items())
    frozen = [n for n, p in t2.model.named_parameters() if not p.requires_grad]
    assert frozen and all(".decoder.lang." in n for n in frozen)
    with pytest.raises(KeyError):
        freeze_modules(t2.model, ["no.such.module"])
    rep = load_pretrained(t2.model, str(tmp_path / "a" / "step_00000002"))           # a directory of weight files
    assert rep["loaded"] == len(sd) and not rep["missing"]
    with pytest.raises(KeyError):
        load_pretrained(t2.model, _save_partial(tmp_path, sd), strict=True)
    s = LRScheduler(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0), "cosine_restarts", 1.0, 0.0, 0, 8, num_cycles=2)
    assert s.lr_at(0) == 1.0 and abs(s.lr_at(2) - 0.5) < 1e-9 and s.lr_at(4) == 1.0 and s.lr_at(8) == 0.0 and s.lr_at(20) == 0.0
    pl = LRScheduler(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0), "polynomial", 1.0, 0.1, 0, 10, power=2.0)
    assert abs(pl.lr_at(5) - (0.1 + 0.9 * 0.25)) < 1e-9
    with pytest.raises(ValueError):
        validate(EmbodiedArgs(optimizer="adagrad"))
    with pytest.raises(ValueError):
        validate(EmbodiedArgs(async_save=True, checkpoint_format="dcp"))


def _save_partial(tmp_path, sd):
    p = str(tmp_path / "partial.pt")
    torch.save({k: v for i, (k, v) in enumerate(sd.items()) if i % 2 == 0}, p)
    return p


def _write_lerobot(root, episodes=2, steps=6, size=(24, 32)):
    """A tiny LeRobot v2 data set: parquet episodes, one mp4 per camera and episode, meta files."""
    import cv2
    import pyarrow as pa
    import pyarrow.parquet as pq

    os.makedirs(root / "meta", exist_ok=True)
    feats = {"observation.images.front": {"dtype": "video"}, "observation.images.wrist": {"dtype": "video"},
             "observation.state": {"dtype": "float32", "shape": [4]}, "action": {"dtype": "float32", "shape": [3]}}
    (root / "meta" / "info.json").write_text(json.dumps({"fps": 10, "robot_type": "toy_arm", "features": feats,
                                                        "video_path": "videos/{episode_chunk_dir}/{video_key}/episode_{episode_index:06d}.mp4"}))
    (root / "meta" / "tasks.jsonl").write_text(json.dumps({"task_index": 0, "task": "stack the blocks"}) + "\n")
    (root / "meta" / "stats.json").write_text(json.dumps({"observation.state": {"mean": [0] * 4, "std": [1] * 4, "min": [-1] * 4, "max": [1] * 4,
                                                                                  "q01": [-1] * 4, "q99": [1] * 4},
                                                          "action": {"mean": [0] * 3, "std": [1] * 3, "min": [-1] * 3, "max": [1] * 3,
                                                                     "q01": [-1] * 3, "q99": [1] * 3}}))
    for e in range(episodes):
        d = root / "data" / "chunk-000"
        os.makedirs(d, exist_ok=True)
        pq.write_table(pa.table({"observation.state": [[float(e), float(t), 0.0, 1.0] for t in range(steps)],
                                 "action": [[0.1 * t, 0.0, float(e)] for t in range(steps)],
                                 "task_index": [0] * steps, "episode_index": [e] * steps}), d / f"episode_{e:06d}.parquet")
        for cam, base in (("observation.images.front", 40), ("observation.images.wrist", 160)):
            vd = root / "videos" / "chunk-000" / cam
            os.makedirs(vd, exist_ok=True)
            w = cv2.VideoWriter(str(vd / f"episode_{e:06d}.mp4"), cv2.VideoWriter_fourcc(*"mp4v"), 10, (size[1], size[0]))
            for t in range(steps):
                w.write(np.full((size[0], size[1], 3), base + 10 * t, np.uint8))
            w.release()


def test_lerobot_v2_dataset_reads_videos_and_meta(tmp_path):
    from loongforge_b200.embodied.data import LeRobotDataset, build_dataset, collate

    root = tmp_path / "ds"
    _write_lerobot(root)
    a = _args(tmp_path / "o", dataset_type="lerobot", dataset_path=str(root), num_cameras=2, image_size=16, action_dim=3, state_dim=4,
              action_horizon=3, video_frames=5, video_frame_stride=1)
    ds = build_dataset(a)
    assert isinstance(ds, LeRobotDataset) and len(ds) == 12 and ds.cameras == ["observation.images.front", "observation.images.wrist"]
    s = ds[8]                                                     # episode 1, step 2
    assert s["images"].shape == (2, 3, 16, 16) and s["state"].tolist() == [1.0, 2.0, 0.0, 1.0]
    front, wrist = s["images"][0].mean() * 255, s["images"][1].mean() * 255
    assert abs(front - 60) < 6 and abs(wrist - 180) < 6            # frame 2 of each camera (lossy codec)
    assert s["actions"].shape == (3, 3) and abs(s["actions"][1, 0] - 0.3) < 1e-6 and s["action_mask"].tolist() == [1, 1, 1]
    assert ds[11]["action_mask"].tolist() == [1, 0, 0]            # last step of the episode: padded chunk
    v = s["video"]
    assert v.shape == (5, 3, 16, 16) and v[1].mean() > v[0].mean() and abs(v[4].mean() - v[3].mean()) < 1e-6   # clamps at the end
    assert ds.stats()["action"]["q99"] == [1, 1, 1]
    only = LeRobotDataset(a, str(root), cameras=["observation.images.wrist"], episodes=[1])
    assert len(only) == 6 and abs(only[0]["images"][0].mean() * 255 - 160) < 6 and only[0]["images"][1].max() == 0
    ds.raw = True
    assert ds[0]["task"] == "stack the blocks" and ds[0]["embodiment_tag"] == "toy_arm"
    b = collate([build_dataset(a)[i] for i in range(2)])
    assert b["video"].shape == (2, 5, 3, 16, 16)
    # statistics of the data set itself feed the transforms
    a2 = _args(tmp_path / "o2", dataset_type="lerobot", dataset_path=str(root), num_cameras=2, image_size=16, action_dim=3, state_dim=4,
               action_horizon=3, use_transforms=True, stats_path=str(root), model_name="groot_n1_6", embodiment_tags={"toy_arm": 5})
    t = build_dataset(a2)[3]
    assert t["embodiment_id"] == 5 and t["images"].shape == (2, 3, 16, 16)


def test_dataset_mixture_proportions(tmp_path):
    from loongforge_b200.embodied.data import MixtureDataset, SyntheticEpisodes, build_dataset, collate

    root = tmp_path / "ds"
    _write_lerobot(root)
    a = _args(tmp_path / "o", num_cameras=2, image_size=16, action_dim=3, state_dim=4, action_horizon=3,
              dataset_mixture=[{"type": "lerobot", "path": str(root), "weight": 3}, {"type": "synthetic", "weight": 1}],
              mixture_epoch_length=400)
    ds = build_dataset(a)
    assert isinstance(ds, MixtureDataset) and len(ds) == 400
    ids = np.array([int(ds[i]["dataset_id"]) for i in range(400)])
    assert 0.68 < (ids == 0).mean() < 0.82                        # 3 : 1
    again = build_dataset(a)
    assert [int(again[i]["dataset_id"]) for i in range(50)] == ids[:50].tolist()      # same seed, same schedule
    firsts = [ds[i]["state"].tolist() for i in np.nonzero(ids == 0)[0][:13]]
    assert firsts[12] == firsts[0]                                # the 12-sample robot set wraps around
    b = collate([ds[i] for i in range(4)])
    assert b["images"].shape == (4, 2, 3, 16, 16) and b["dataset_id"].shape == (4,)


def test_microbatch_graph_runner_signatures_and_padding():
    """On CPU the runner is eager, but its bookkeeping is the same: token fields padded to the configured multiple, one slot
    per input signature, least recently used slot dropped, gradients accumulated with the given scale."""
    from loongforge_b200.embodied.cuda_graph import MicrobatchGraphRunner, pad_batch, shape_key

    b = {"text": torch.ones(2, 5, dtype=torch.long), "state": torch.zeros(2, 3)}
    p = pad_batch(b, 8)
    assert p["text"].shape == (2, 8) and p["text"][:, 5:].sum() == 0 and p["state"] is b["state"]
    assert shape_key(p) != shape_key(b) and shape_key(pad_batch({"text": torch.ones(2, 7, dtype=torch.long), "state": torch.zeros(2, 3)}, 8)) == shape_key(p)
    lin = torch.nn.Linear(3, 1)
    loss_fn = lambda m, batch: m(batch["state"]).pow(2).mean() + 0 * batch["text"].float().mean()  # noqa: E731
    r = MicrobatchGraphRunner(lin, loss_fn, warmup=1, pad_to=8, max_graphs=2)
    x = torch.randn(2, 3)
    l1 = r.run({"text": torch.ones(2, 5, dtype=torch.long), "state": x}, scale=0.5)
    g1 = lin.weight.grad.clone()
    ref = torch.nn.Linear(3, 1)
    ref.load_state_dict(lin.state_dict())
    (0.5 * ref(x).pow(2).mean()).backward()
    assert torch.allclose(g1, ref.weight.grad) and torch.allclose(l1, ref(x).pow(2).mean())
    r.run({"text": torch.ones(2, 7, dtype=torch.long), "state": x}, scale=0.5)          # same signature after padding
    assert len(r.captured) == 1 and next(iter(r.captured.values())).calls == 2
    assert torch.allclose(lin.weight.grad, 2 * g1)                                        # accumulated
    r.run({"text": torch.ones(2, 9, dtype=torch.long), "state": x})
    r.run({"text": torch.ones(2, 17, dtype=torch.long), "state": x})
    assert len(r.captured) == 2 and r.calls == 4 and r.graph is None                      # oldest signature dropped; no GPU: eager


def test_hdf5_bimanual_episodes(tmp_path):
    """Trajectory logic of the HDF5 data set on a dictionary-backed episode (no HDF5 library needed): rotation layout
    against SciPy, two-second windows on the common clock, static windows dropped, first point = state."""
    import json
    import numpy as np
    from scipy.spatial.transform import Rotation

    from loongforge_b200.embodied.config import EmbodiedArgs
    from loongforge_b200.embodied.hdf5_data import HDF5Episodes, arm_trajectories, quat_xyzw_to_rot6d

    rng = np.random.default_rng(0)
    q = rng.normal(size=(5, 4))
    want = Rotation.from_quat(q / np.linalg.norm(q, axis=-1, keepdims=True)).as_matrix()[..., :, :2].reshape(5, 6)
    assert np.allclose(quat_xyzw_to_rot6d(q), want, atol=1e-9)

    T = 120
    eef = np.zeros((T, 16), dtype=np.float32)
    eef[:, 6] = eef[:, 14] = 1.0                                   # identity rotations
    t = np.arange(T) / 30.0
    eef[60:, 0] = t[60:] - t[60]                                   # the left arm rests for two seconds, then moves
    eef[:, 7], eef[:, 15] = 0.01, 0.05                             # left gripper closed (0.5 < 1), right open
    left, right = arm_trajectories(eef)
    assert left.shape == (T, 10) and left[0, 9] == 1.0 and right[0, 9] == 0.0 and np.allclose(left[0, 3:9], [1, 0, 0, 1, 0, 0])
    store = {"observations/eef_quaternion": eef, "language_instruction": b"fold the towel",
             "observations/images/cam_high": rng.integers(0, 255, size=(T, 12, 16, 3), dtype=np.uint8)}
    (tmp_path / "metadata.json").write_text(json.dumps({"dataset_name": "agilex", "datalist": ["episode_0.hdf5"],
                                                        "observation_key": ["observations/images/cam_high"]}))
    a = EmbodiedArgs(model_name="xvla", action_horizon=8, image_size=8, num_cameras=2, max_text_len=8)
    ds = HDF5Episodes(a, str(tmp_path), opener=lambda path: store)
    starts = [s for _, s in ds.index]
    assert starts and all(s % 2 == 0 and s < T - 30 for s in starts)
    assert min(starts) > 0 and min(starts) <= 60                   # the windows before any motion are dropped
    s = ds[0]
    assert s["images"].shape == (2, 3, 8, 8) and s["images"][1].max() == 0 and 0 <= s["images"][0].min() and s["images"][0].max() <= 1
    assert s["state"].shape == (20,) and s["actions"].shape == (8, 20) and s["action_mask"].sum() == 8
    i = starts.index(60)
    w = ds[i]
    assert np.allclose(w["state"][0], 0.0) and np.allclose(w["actions"][-1][0], 59 / 30, atol=1e-5)   # held at the episode's end
    assert np.allclose(np.diff(w["actions"][:, 0])[:3], (59 / 30) / 8, atol=1e-4)
    ds.raw = True
    assert ds[0]["task"] == "fold the towel" and ds[0]["embodiment_tag"] == "agilex"
    assert ds.__getstate__()["_open"] == {} and ds._open        # open files stay out of what loader workers receive


def test_merge_stats_and_block_shard_sampler(tmp_path):
    import json
    import numpy as np
    from loongforge_b200.embodied.data import BlockShardSampler
    from loongforge_b200.embodied.transforms import compute_stats, load_stats, merge_stats

    rng = np.random.default_rng(0)
    parts = [rng.normal(i, 1 + i, size=(50 + 20 * i, 3)) for i in range(3)]
    merged = merge_stats([{"action": compute_stats([p])} for p in parts])["action"]
    whole = compute_stats([np.concatenate(parts)])
    for k in ("mean", "std", "min", "max"):
        assert np.allclose(merged[k], whole[k], atol=1e-9), k
    assert merged["count"] == [210] and np.all(np.asarray(merged["q99"]) >= np.asarray(whole["q99"]))
    (tmp_path / "meta").mkdir()
    with open(tmp_path / "meta" / "episodes_stats.jsonl", "w") as f:
        for i, p in enumerate(parts):
            f.write(json.dumps({"episode_index": i, "stats": {"action": compute_stats([p])}}) + "\n")
    assert np.allclose(load_stats(str(tmp_path))["action"]["std"], whole["std"], atol=1e-9)

    data = list(range(23))
    one = list(BlockShardSampler(data, 2, 1, 0, seed=5))
    ranks = [list(BlockShardSampler(data, 2, 2, r, seed=5)) for r in range(2)]
    assert len(ranks[0]) == len(ranks[1]) == 10 == len(BlockShardSampler(data, 2, 2, 0))
    for k in range(5):                                            # round k on two ranks = batches 2k, 2k+1 of one process
        assert ranks[0][2 * k:2 * k + 2] == one[4 * k:4 * k + 2] and ranks[1][2 * k:2 * k + 2] == one[4 * k + 2:4 * k + 4]
    s = BlockShardSampler(data, 2, 2, 0, seed=5)
    s.set_epoch(1)
    assert list(s) != ranks[0]


def test_export_checkpoint_folds_lora_into_one_file(tmp_path):
    """A LoRA run's checkpoint exported to one safetensors file loads into a plain model and gives the same loss."""
    from safetensors.torch import load_file

    from loongforge_b200.embodied import export_checkpoint as ex
    from loongforge_b200.embodied.models import build_policy
    from loongforge_b200.embodied.trainer import build_trainer

    a = _args(tmp_path, lora_rank=2, lora_targets=["qkv", "o"], train_steps=2, save_interval=2, lr=1e-2)
    t = build_trainer(a)
    t._setup()
    _open_gates(t.model)
    t._training_loop()
    assert any(float(p.abs().max()) > 0 for n, p in t.model.named_parameters() if ".lora_b." in n)   # something to fold
    root = os.path.join(a.output_dir, "checkpoints")
    root = root if os.path.isdir(root) else a.output_dir
    out = str(tmp_path / "release" / "policy.safetensors")
    assert ex.main(["--ckpt", root, "--out", out]) == 0
    sd = load_file(out)
    assert sd and not any("lora_" in k or ".base." in k for k in sd)
    plain = build_policy(a.model_name, a)
    missing, unexpected = plain.load_state_dict(sd, strict=False)
    assert not unexpected and not missing
    batch = next(iter(t.loader))
    t.model.eval(), plain.eval()
    with torch.no_grad():
        torch.manual_seed(3)
        want = float(t.model(batch))
        torch.manual_seed(3)
        got = float(plain(batch))
    assert abs(want - got) < 1e-5 * max(1.0, abs(want))
    kept = ex.export(root, str(tmp_path / "kept.pt"), fmt="pt", keep_lora=True, dtype="bf16")
    blob = torch.load(str(tmp_path / "kept.pt"))
    assert kept["lora_folded"] == 0 and any(".lora_a." in k for k in blob) and all(
        v.dtype == torch.bfloat16 for v in blob.values() if v.is_floating_point())


def test_video_backends_decode_by_index_and_time(tmp_path):
    import cv2
    from loongforge_b200.embodied.video_backends import decode_frames

    path = str(tmp_path / "clip.mp4")
    w = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 10.0, (32, 32))
    for i in range(10):
        w.write(np.full((32, 32, 3), i * 25, dtype=np.uint8))
    w.release()
    got = decode_frames(path, indices=[7, 2, 2, 9, 30])
    assert got.shape == (5, 32, 32, 3) and got.dtype == np.uint8
    level = got.reshape(5, -1).mean(1)
    assert np.allclose(level, [175, 50, 50, 225, 225], atol=6)        # request order kept, past the end = last frame
    by_time = decode_frames(path, timestamps=[0.0, 0.31, 0.7]).reshape(3, -1).mean(1)
    assert np.allclose(by_time, [0, 75, 175], atol=6)
    with pytest.raises(ValueError):
        decode_frames(path)
    with pytest.raises(ValueError):
        decode_frames(path, indices=[0], backend="vhs")
    with pytest.raises(ImportError, match="not installed"):
        decode_frames(path, indices=[0], backend="decord")
