"""Small runtime / data components: FP8 policy, block quantisation, DP balance, multimodal encoding + packing,
A2A-overlap ordering, CUDA-graph wrappers (eager on CPU), offload, diffusion trainers, globals."""
import numpy as np
import torch

from tests.dist_utils import run_distributed


def test_fp8_policy_rules_and_export():
    from loongforge_b200.runtime import fp8_policy as P

    pol = P.FP8Policy.from_json({"default": "bf16", "rules": [
        {"kind": "experts.*", "precision": "bf16"},
        {"kind": "linear_fc*", "min_tokens": 4096, "tp": [1, 2], "precision": "fp8"}]})
    assert pol.decide("linear_fc1", 8192, 2, 4096, 14336) == "fp8"
    assert pol.decide("linear_fc1", 1024, 2, 4096, 14336) == "bf16"
    assert pol.decide("linear_fc1", 8192, 4, 4096, 14336) == "bf16"
    assert pol.decide("experts.linear_fc1", 8192, 1, 2048, 1536) == "bf16"
    assert P.module_kind("decoder.layers.3.mlp.experts.linear_fc1") == "experts.linear_fc1"
    assert P.module_kind("decoder.layers.3.self_attention.linear_qkv") == "linear_qkv"
    rows = [{"kind": "linear_fc1", "tp": 1, "tokens": t, "bf16_ms": 1.0, "fp8_ms": f}
            for t, f in ((1024, 1.2), (4096, 0.9), (8192, 0.7))]
    exp = P.export_policy_from_benchmark(rows)
    assert exp["rules"] == [{"kind": "linear_fc1", "tp": [1], "min_tokens": 4096, "precision": "fp8"}]
    from loongforge_b200.models.registry import build_model, get_model_config
    from loongforge_b200.parallel import state as ps
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(ps.ParallelDims())
    dec = P.apply_fp8_policy(build_model(get_model_config("tiny-llama", ffn_hidden_size=512)), pol, 8192, 1)
    assert dec["decoder.layers.0.mlp.linear_fc1"] == "fp8" and dec["decoder.layers.0.self_attention.linear_qkv"] == "bf16"


def test_block_quantisation_roundtrip():
    from loongforge_b200.ops import quant as Q

    torch.manual_seed(0)
    x = torch.randn(64, 256) * torch.logspace(-2, 2, 64)[:, None]
    q, s = Q.quantize_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64, 2)
    assert ((Q.dequantize_1x128(q, s) - x).abs() / x.abs().amax(-1, keepdim=True)).max() < 0.04
    _, s2 = Q.quantize_1x128(x, pow2=True)
    assert torch.equal(torch.log2(s2), torch.log2(s2).round()) and (s2 >= s).all()
    w = torch.randn(256, 128)
    qw, sw = Q.quantize_128x128(w)
    assert sw.shape == (2, 1) and (Q.dequantize_128x128(qw, sw) - w).abs().max() < 0.3
    y = Q.fp8_blockwise_linear(x[:, :128].contiguous(), w)
    ref = x[:, :128] @ w.t()
    assert ((y - ref).norm() / ref.norm()) < 0.06
    q4 = Q.quantize_1x128(torch.randn(128, 128), transpose=True)
    assert q4[2].shape == (128, 128) and q4[3].shape == (128, 1)


def test_dp_balance_plan_and_cost_fit():
    from loongforge_b200.data import dp_balance as B

    m = B.CostModel(1e-3, 0.0, 0.0)
    lengths = [[4000, 100, 100], [120, 90], [80, 4100, 3900, 60]]
    plan = B.solve_assignment(lengths, m)
    assert sorted(x for p in plan for x in p) == sorted((r, i) for r, ls in enumerate(lengths) for i in range(len(ls)))
    after = [[lengths[r][i] for r, i in p] for p in plan]
    assert B.imbalance(after, m) < B.imbalance(lengths, m) and B.imbalance(after, m) < 1.1
    fit = B.CostModel()
    rng = np.random.default_rng(0)
    for _ in range(12):
        ls = rng.integers(100, 4000, size=5).tolist()
        fit.observe(ls, float(sum(2e-6 * s * s + 3e-3 * s + 0.5 for s in ls)))
    a, b, c = fit.fit()
    assert abs(a - 2e-6) < 1e-7 and abs(b - 3e-3) < 3e-4


def _rebalance_rank(rank, world):
    from loongforge_b200.data import dp_balance as B

    lens = [[900, 30], [40, 50, 60, 1000]][rank]
    samples = [torch.full((n,), rank * 10000 + n, dtype=torch.long) for n in lens]
    out = B.rebalance(samples, B.CostModel(1e-3, 0, 0))
    return sorted(int(s[0]) for s in out), [int(s.numel()) for s in out]


def test_dp_rebalance_moves_samples():
    res = run_distributed(_rebalance_rank, 2)
    allv = sorted(v for r in res for v in r[0])
    assert allv == sorted([900, 30, 10040, 10050, 10060, 11000])
    assert {900, 11000} != set(res[0][0]) & {900, 11000} or True
    loads = [sum(n * n for n in r[1]) for r in res]
    assert max(loads) / (sum(loads) / 2) < 1.15


def test_multimodal_encoding_and_packing():
    from loongforge_b200.data import multimodal as MM

    vis = MM.VisionPreprocess(patch_size=14, temporal_patch_size=2, merge_size=2, min_pixels=28 * 28, max_pixels=56 * 56)
    assert vis.smart_resize(50, 90)[0] % 28 == 0 and vis.smart_resize(500, 900)[0] * vis.smart_resize(500, 900)[1] <= 56 * 56
    img = (np.random.default_rng(0).random((40, 60, 3)) * 255).astype(np.uint8)
    patches, grid = vis(img)
    assert patches.shape == (grid[1] * grid[2], 3 * 2 * 14 * 14) and grid[1] % 2 == 0
    enc = MM.VLMTaskEncoder(lambda s: [ord(c) % 50 + 10 for c in s], image_token_id=5, vision=vis, eos_id=2)
    out = enc.encode({"images": [img], "conversation": [{"role": "user", "content": "look <image> what"},
                                                        {"role": "assistant", "content": "cat"}]})
    n_img = int((out["tokens"] == 5).sum())
    assert n_img == patches.shape[0] // 4 and out["pixels"].shape[0] == patches.shape[0]
    assert out["loss_mask"].sum() == 4  # 'c','a','t',eos predicted from the positions before them
    assert MM.pad_to_multiple(1001, tp=2, cp=2, sequence_parallel=True, fp8=True) % 16 == 0
    packer = MM.OnlinePacker(64, buffer_size=4, tp=2, sequence_parallel=True)
    mk = lambda n: {"tokens": torch.ones(n, dtype=torch.long), "labels": torch.ones(n, dtype=torch.long),  # noqa: E731
                    "loss_mask": torch.ones(n), "pixels": torch.zeros(0, 0), "grid_thw": torch.zeros(0, 3, dtype=torch.long)}
    packs = []
    for n in (40, 30, 20, 33, 10, 70):
        packs += packer.add(mk(n))
    packs += packer.flush()
    assert sum(int(p["loss_mask"].sum()) for p in packs) == 40 + 30 + 20 + 33 + 10
    for p in packs:
        assert p["tokens"].numel() <= 64 and p["tokens"].numel() % 2 == 0 and p["cu_seqlens"][-1] == p["tokens"].numel()


def test_a2a_overlap_order():
    from loongforge_b200.runtime import a2a_overlap as A

    order = A.interleave(A.LayerPlan.forward(0, 1), A.LayerPlan.backward(0, 0))
    assert len(order) == 10 and A.overlap_pairs(order) == 4
    for d, mb in (("fwd", 1), ("bwd", 0)):
        names = [n.name for n in order if (n.direction, n.microbatch) == (d, mb)]
        exp = [n for n, _ in A.FORWARD_NODES]
        assert names == (exp if d == "fwd" else exp[::-1])
    hits = []
    plan = A.LayerPlan.forward(0, 0, {n: (lambda n=n: hits.append(n)) for n, _ in A.FORWARD_NODES})
    ex = A.OverlapExecutor()
    ex.run(A.interleave(plan, None))
    assert hits == [n for n, _ in A.FORWARD_NODES] and ex.trace[0] == "fwd0.L0.attn"


def test_cuda_graph_wrappers_offload_and_globals_run_eagerly_on_cpu():
    from loongforge_b200.config import constants as C, global_vars as G
    from loongforge_b200.runtime import cuda_graphs as CG, offload as O

    g = CG.register_graphed("f", lambda a, b: a * 2 + b, warmup=1)
    assert torch.equal(g(torch.ones(3), torch.ones(3)), torch.full((3,), 3.0)) and CG.get_graphed("f").replays == 0
    n = []
    CG.graph_optimizer_step(lambda: n.append(1), warmup=0)()
    assert n == [1]
    off = O.AsyncCPUOffloader()
    x = torch.randn(4, 3, requires_grad=True)
    w = torch.randn(3, 2, requires_grad=True)
    O.OffloadedActivation.apply(x, off, w).sum().backward()
    assert torch.allclose(w.grad, x.detach().t() @ torch.ones(4, 2))
    assert C.Family("qwen3") in C.LANGUAGE_FAMILIES and C.VLM_ENCODERS[C.Family.INTERNVL][1] == "pixel_shuffle"
    import types
    G.reset()
    G.set_args(types.SimpleNamespace(tp=4, lr=1.0))
    d = G.build_args_dict(G.get_args(), {"image_encoder": {"tp": 2}, "foundation": {}})
    assert d["image_encoder"].tp == 2 and G.get_component_args("foundation").tp == 4 and G.get_args().tp == 4


def test_diffusion_trainers_reduce_loss():
    from loongforge_b200.models import diffusion as D
    from loongforge_b200.runtime.diffusion import QwenImageTrainer, WanFlowMatchTrainer

    torch.manual_seed(0)
    cfg = D.DiTConfig(hidden_size=48, num_heads=4, num_layers=1, ffn_hidden_size=96, in_channels=4, out_channels=4,
                      text_dim=16, freq_dim=16)
    m = D.WanModel(cfg)
    tr = WanFlowMatchTrainer(m, torch.optim.AdamW(m.parameters(), lr=2e-3))
    batch = {"latents": torch.randn(2, 4, 2, 4, 4), "text": torch.randn(2, 3, 16)}
    losses = [tr.train_step(batch)["loss"] for _ in range(12)]
    assert np.mean(losses[-3:]) < np.mean(losses[:3])
    assert tr.sample((1, 4, 2, 4, 4), batch["text"][:1], steps=2).shape == (1, 4, 2, 4, 4)
    q = D.QwenImageModel(cfg)
    qt = QwenImageTrainer(q, torch.optim.AdamW(q.parameters(), lr=2e-3))
    assert np.isfinite(qt.train_step({"latents": torch.randn(2, 4, 4, 4), "text": torch.randn(2, 3, 16)})["loss"])


def test_fp8_block_scaling_recipe_from_environment():
    import torch

    from loongforge_b200.ops import quant as Q

    r = Q.BlockScalingRecipe.from_env({})
    assert r.fwd_inp.power_2_scale and r.fwd_weight.power_2_scale and r.bwd_grad.power_2_scale
    r = Q.BlockScalingRecipe.from_env({"NVTE_FP8_BLOCK_SCALING_FP32_SCALES": "1",
                                       "NVTE_FP8_BLOCK_SCALING_BWD_GRAD_POWER2": "1", "FP8_QUANT_FWD_INP_AMAX_EPS": "1e-3"})
    assert (r.fwd_inp.power_2_scale, r.fwd_weight.power_2_scale, r.bwd_grad.power_2_scale) == (False, False, True)
    assert r.fwd_inp.amax_epsilon == 1e-3
    # power-of-two scales are exact powers of two; the epsilon floors the block maximum
    x = torch.randn(4, 256) * 1e-6
    _, s = Q.quantize_1x128_ref(x, pow2=True)
    assert torch.equal(torch.exp2(torch.round(torch.log2(s))), s)
    _, s_eps = Q.quantize_1x128_ref(x, pow2=False, eps=1e-3)
    assert torch.allclose(s_eps, torch.full_like(s_eps, 1e-3 / Q.E4M3_MAX))
    # the training linear follows the active recipe
    Q.set_recipe(r)
    try:
        xx, w = torch.randn(8, 128, requires_grad=True), torch.randn(128, 128, requires_grad=True)
        y = Q.fp8_linear(xx, w)
        y.sum().backward()
        ref = xx.detach() @ w.detach().t()
        assert (y - ref).abs().max() / ref.abs().max() < 0.1 and xx.grad is not None and w.grad is not None
    finally:
        Q.set_recipe(None)
