"""World-model policies of the embodied stack (LingBot-VA, FastWAM, DreamZero, Cosmos3) and their shared parts: the
causal latent codec, attention masks, and the property that makes each of them usable as a policy — what the network
computes for one step under teacher forcing is what it computes in the test-time layout (roll-out, cached first frame,
packed row)."""
import pytest
import torch

from loongforge_b200.embodied.config import EmbodiedArgs, validate


def _batch(B=2, frames=5, size=32, horizon=4, adim=7):
    torch.manual_seed(1)
    return dict(images=torch.rand(B, 1, 3, size, size), video=torch.rand(B, frames, 3, size, size),
                text=torch.tensor([[5, 6, 7, 0, 0, 0], [8, 9, 10, 11, 12, 0]])[:B], state=torch.randn(B, 8),
                actions=torch.randn(B, horizon, adim).clamp(-1, 1), action_mask=torch.ones(B, horizon))


def test_causal_video_codec_shapes_and_causality():
    from loongforge_b200.embodied.wan_blocks import CausalVideoVAE

    torch.manual_seed(0)
    vae = CausalVideoVAE(z_dim=8, base=8)
    v = torch.randn(2, 3, 9, 32, 32)
    z = vae.encode(v)
    assert z.shape == (2, 8, 3, 4, 4) and vae.latent_frames(9) == 3
    assert vae.decode(z).shape == v.shape
    v2 = v.clone()
    v2[:, :, 5:] += 1.0                                   # frames 5.. belong to the third latent frame only
    z2 = vae.encode(v2)
    assert torch.equal(z2[:, :, :2], z[:, :, :2]) and not torch.allclose(z2[:, :, 2], z[:, :, 2])
    z3 = torch.cat([z[:, :, :2], z[:, :, 2:] + 1], dim=2)
    r, r3 = vae.decode(z), vae.decode(z3)
    assert torch.equal(r[:, :, :5], r3[:, :, :5]) and not torch.allclose(r[:, :, 5:], r3[:, :, 5:])
    with pytest.raises(AssertionError):
        vae.encode(torch.randn(1, 3, 8, 32, 32))


def test_flow_schedule_tables():
    from loongforge_b200.embodied.wan_blocks import FlowSchedule

    s = FlowSchedule(1000, shift=5.0)
    assert s.sigmas[0] == 1.0 and (s.sigmas[1:] < s.sigmas[:-1]).all() and s.sigmas[-1] > 0
    ids = torch.tensor([[0, 999], [500, 250]])
    x0, noise = torch.zeros(2, 2, 3), torch.ones(2, 2, 3)
    assert torch.allclose(s.add_noise(x0, noise, ids, 1)[..., 0], s.sigmas[ids])
    assert abs(s.weights.sum().item() - 1000) < 1e-2 and s.weights.min() == 0
    inf = s.inference_sigmas(4)
    assert inf[0] == 1 and inf[-1] == 0 and inf.numel() == 5
    beta = s.sample_ids((4000,), beta=(3.0, 1.0))
    assert beta.float().mean() < 400                      # high noise = low id


def test_lingbot_mask_rules():
    from loongforge_b200.embodied.lingbot_va import teacher_forcing_mask

    # two latent chunks (orders 0, 2), two action chunks (1, 3); noisy copies first
    order = torch.tensor([0, 2, 0, 2, 1, 3, 1, 3])
    noisy = torch.tensor([1, 1, 0, 0, 1, 1, 0, 0]).bool()
    m = teacher_forcing_mask(order, noisy, window=10)
    assert m[0].tolist() == [1, 0, 0, 0, 0, 0, 0, 0]      # noisy latent 0: itself only
    assert m[1].tolist() == [0, 1, 1, 0, 0, 0, 1, 0]      # noisy latent 1: itself, clean latent 0, clean action 0
    assert m[4].tolist() == [0, 0, 1, 0, 1, 0, 0, 0]      # noisy action 0: itself, clean latent 0
    assert m[5].tolist() == [0, 0, 1, 1, 0, 1, 1, 0]      # noisy action 1: clean latents 0, 1, clean action 0, itself
    assert m[3].tolist() == [0, 0, 1, 1, 0, 0, 1, 0]      # clean latent 1: clean history, never noisy tokens
    w = teacher_forcing_mask(order, noisy, window=1)
    assert w[5].tolist() == [0, 0, 0, 1, 0, 1, 0, 0]      # window 1: only order 2 (and itself) remain for order 3


def test_lingbot_teacher_forcing_equals_rollout_layout():
    from loongforge_b200.embodied.lingbot_va import LingBotVAConfig, LingBotVAPolicy

    torch.manual_seed(0)
    c = LingBotVAConfig.tiny(action_dim=7)
    p = LingBotVAPolicy(c).eval()
    m = p.model
    B, Fr, n = 2, 3, 2
    lat, act = torch.randn(B, 8, Fr, 4, 4), torch.randn(B, Fr, n, 8)
    nl, na = torch.randn_like(lat), torch.randn_like(act)
    tl, ta = torch.tensor([[900., 500., 100.]]).expand(B, -1), torch.tensor([[300., 600., 800.]]).expand(B, -1)
    zero = torch.zeros(B, Fr)
    text = torch.randn(B, 4, c.text_dim)
    with torch.no_grad():
        full = m([m.latent_part(nl, tl, True, 1), m.latent_part(lat, zero, False, 1),
                  m.action_part(na, ta, True, 1), m.action_part(act, zero, False, 1)], text, window=64)
        # step 1 alone: clean latents 0..1 and clean actions 0 are the history of noisy action chunk 1
        roll = m([m.latent_part(lat[:, :, :2], zero[:, :2], False, 1), m.action_part(act[:, :1], zero[:, :1], False, 1),
                  m.action_part(na[:, 1:2], ta[:, 1:2], True, 1, first_frame=1)], text, window=64)
        # and latent frame 2 given clean latents 0..1 and clean actions 0..1
        roll_l = m([m.latent_part(lat[:, :, :2], zero[:, :2], False, 1), m.action_part(act[:, :2], zero[:, :2], False, 1),
                    m.latent_part(nl[:, :, 2:], tl[:, 2:], True, 1, first_frame=2)], text, window=64)
    assert torch.allclose(full[2][:, n:2 * n], roll[-1], atol=1e-5)
    assert torch.allclose(full[0][:, 2 * 4:], roll_l[-1], atol=1e-5)


def test_fastwam_masks_and_cached_first_frame():
    from loongforge_b200.embodied.fastwam import FastWAMConfig, FastWAMPolicy, mot_mask, video_to_video_mask
    from loongforge_b200.embodied.wan_blocks import video_from_batch

    vv = video_to_video_mask(3, 2, "first_frame_causal")
    assert not vv[:2, 2:].any() and vv[2:].all() and vv[:2, :2].all()
    assert video_to_video_mask(3, 2, "per_frame_causal")[2:4].tolist() == [[1, 1, 1, 1, 0, 0]] * 2
    f = mot_mask("fastwam", 3, 2, 2, "first_frame_causal")
    assert f[6:, :2].all() and not f[6:, 2:6].any() and f[6:, 6:].all() and not f[:6, 6:].any()
    assert mot_mask("joint", 3, 2, 2, "first_frame_causal")[6:].all()
    i = mot_mask("idm", 2, 2, 3, "bidirectional")
    assert i.shape == (11, 11) and i[8:, 4:8].all() and not i[8:, :4].any() and not i[:4, 4:8].any()

    torch.manual_seed(0)
    batch = _batch()
    c = FastWAMConfig.tiny(action_dim=7)
    p = FastWAMPolicy(c).eval()
    m = p.model
    with torch.no_grad():
        first = p.vae.encode(video_from_batch(batch, 1)[:, :, :1])
        text, tm = p._text(batch)
        a, t = torch.randn(2, 4, 7), torch.full((2,), 500.0)
        cache = p.prefill_video_cache(first, text, tm, batch["state"])
        ctx, cm = m.context(text, tm, batch["state"])
        x, mod, ang = m.embed_action(a, t)
        cached = m.layers([dict(expert=m.action, x=x, mod=mod, angles=ang, ctx=m.action.text_embedding(ctx), ctx_mask=cm)],
                          torch.ones(4, cache[0][0].shape[1] + 4, dtype=torch.bool), cache=cache)[0]
        lat = torch.cat([first, torch.randn(2, 8, 1, 4, 4)], dim=2)        # any later frame: actions must not see it
        xv, modv, _, angv, grid = m.embed_video(lat, torch.full((2,), 300.0))
        joint = m.layers(p._streams(text, tm, batch["state"], [(xv, modv, angv)], m.embed_action(a, t)),
                         mot_mask("fastwam", 2, 4, 4, "first_frame_causal"))[-1]
    assert torch.allclose(cached, joint, atol=1e-5)


def test_dreamzero_mask_and_teacher_forcing_equals_rollout():
    from loongforge_b200.embodied.dreamzero import DreamZeroConfig, DreamZeroPolicy, block_causal_mask

    # 3 frames of 1 token, 1 frame per block, 1 action + 1 state per block: [c0 c1 c2 | n0 n1 n2 | a0 a1 | s0 s1]
    m = block_causal_mask(3, 1, 1, 2, 1, 2, 1, True).int().tolist()
    assert m[0] == [1, 0, 0, 0, 0, 0, 0, 0, 0, 0] and m[2] == [1, 1, 1, 0, 0, 0, 0, 0, 0, 0]
    assert m[3] == [0, 0, 0, 1, 0, 0, 0, 0, 0, 0]          # noisy observation: itself
    assert m[5] == [1, 1, 0, 0, 0, 1, 0, 1, 0, 1]          # noisy block 1: clean obs + block 0, itself, its action / state
    assert m[7] == [1, 1, 0, 0, 0, 1, 0, 1, 0, 1]          # action of block 1
    assert m[9] == [0, 0, 0, 0, 0, 0, 0, 0, 0, 1]          # state: itself
    w = block_causal_mask(4, 1, 1, 3, 1, 3, 1, True, local_blocks=1).int().tolist()
    assert w[4 + 3][:4] == [1, 0, 1, 0]                    # noisy block 2 with a one-block window: observation + block 1

    torch.manual_seed(0)
    c = DreamZeroConfig.tiny(action_dim=7)
    p = DreamZeroPolicy(c).eval()
    net = p.model
    B = 2
    lat, noisy = torch.randn(B, 8, 3, 4, 4), torch.randn(B, 8, 3, 4, 4)
    text, img = torch.randn(B, 5, 32), torch.randn(B, 17, 24)
    act, st = torch.randn(B, 4, 8), torch.randn(B, 2, 8)
    t_frame = torch.tensor([[100., 400., 700.]]).expand(B, -1)
    t_act = torch.tensor([[400., 400., 700., 700.]]).expand(B, -1)
    with torch.no_grad():
        vv, av = net(noisy, t_frame, lat[:, :, :1], text, img, act, t_act, st, clean_video=lat)
        hist = torch.cat([lat[:, :, :2], noisy[:, :, 2:]], dim=2)
        vr, ar = net(hist, torch.tensor([[0., 0., 700.]]).expand(B, -1), lat[:, :, :1], text, img, act[:, 2:], t_act[:, 2:],
                     st[:, 1:], register_block_offset=1)
    assert torch.allclose(vv[:, :, 2], vr[:, :, 2], atol=1e-5) and torch.allclose(av[:, 2:], ar, atol=1e-5)
    # embodiment-specific projector: another id gives another action prediction
    with torch.no_grad():
        _, a0 = net(noisy, t_frame, lat[:, :, :1], text, img, act, t_act, st, torch.tensor([0, 0]), clean_video=lat)
        _, a1 = net(noisy, t_frame, lat[:, :, :1], text, img, act, t_act, st, torch.tensor([1, 1]), clean_video=lat)
    assert not torch.allclose(a0, a1)
    p.set_trainable_parameters(tune_projector=True, tune_diffusion_model=False)
    names = [n for n, q in p.model.named_parameters() if q.requires_grad]
    assert names and all(n.startswith(("action_encoder.", "state_encoder.", "action_decoder.")) for n in names)


def test_cosmos3_packing_isolates_samples_and_positions():
    from loongforge_b200.embodied.cosmos3 import (Cosmos3Config, Cosmos3Policy, mrope_angles, pack_samples,
                                                  packed_attention_mask)

    seq = pack_samples([torch.tensor([1, 2]), torch.tensor([3])], [(2, 1, 2), (2, 1, 1)], [2, 1])
    assert seq.length == 12 and seq.sample.tolist() == [0] * 8 + [1] * 4
    assert seq.frame.tolist() == [-1, -1, 0, 0, 1, 1, 1, 1, -1, 0, 1, 1]
    assert seq.position[:, 0].tolist() == [0, 1, 2, 2, 3, 3, 2.5, 3.0, 0, 1, 2, 1.5]      # actions between frames
    m = packed_attention_mask(seq, temporal_causal=True).int()
    assert m[1, :2].tolist() == [1, 1] and m[0, 1] == 0                                     # causal text
    assert m[2].tolist() == [1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0, 0]                             # frame 0: text + frame 0
    assert not m[:8, 8:].any() and not m[8:, :8].any()                                      # samples are isolated
    assert packed_attention_mask(seq, False)[2, :8].all()
    ang = mrope_angles(torch.tensor([[5.0, 1.0, 2.0]]), 12, 10000.0, (2, 2, 2))[0]
    inv = 10000.0 ** (-torch.arange(6) / 6)
    assert torch.allclose(ang, torch.tensor([5.0, 1.0, 2.0, 5.0, 1.0, 2.0]) * inv)

    torch.manual_seed(0)
    c = Cosmos3Config.tiny(action_dim=7)
    p = Cosmos3Policy(c).eval()
    net = p.net
    lats = [torch.randn(8, 2, 4, 4), torch.randn(8, 2, 4, 4)]
    acts = [torch.randn(4, 8), torch.randn(4, 8)]
    texts = [torch.tensor([5, 6, 7]), torch.tensor([8, 9, 10, 11, 12])]
    dom, sig = torch.tensor([0, 2]), torch.tensor([0.3, 0.8])

    def run(ix):
        s = pack_samples([texts[i] for i in ix], [(2, 2, 2)] * len(ix), [4] * len(ix))
        nv = torch.tensor([False] * 4 + [True] * 4).repeat(len(ix))
        with torch.no_grad():
            return net(s, [lats[i] for i in ix], [acts[i] for i in ix], sig[ix], dom[ix], nv, torch.ones(4 * len(ix), dtype=torch.bool))

    both, one = run([0, 1]), run([1])
    assert torch.allclose(both[0][1], one[0][0], atol=1e-5) and torch.allclose(both[1][1], one[1][0], atol=1e-5)


@pytest.mark.parametrize("name,extra", [("lingbot_va", {}), ("fastwam", {"variant": "joint"}), ("fastwam", {"variant": "idm"}),
                                        ("dreamzero", {"decouple_video_action_noise": True, "high_noise_beta": (3.0, 1.0)}),
                                        ("cosmos3", {"video_temporal_causal": True, "predict_text_tokens": True})])
def test_world_model_policies_train_on_future_frames(name, extra, tmp_path):
    """Through the factory and the data set with ``video_frames``: loss decreases over a few steps of Adam."""
    from loongforge_b200.embodied.data import SyntheticEpisodes, collate
    from loongforge_b200.embodied.models import build_policy

    a = validate(EmbodiedArgs(model_name=name, model_overrides=dict(size="tiny", **extra), image_size=32, action_horizon=4,
                              video_frames=9 if name == "dreamzero" else 5, video_frame_stride=2, output_dir=str(tmp_path)))
    torch.manual_seed(0)
    p = build_policy(name, a)
    ds = SyntheticEpisodes(a)
    batch = collate([ds[i] for i in range(2)])
    assert batch["video"].shape == (2, a.video_frames, 3, 32, 32)
    assert not torch.equal(batch["video"][:, 0], batch["video"][:, 1])    # frames move
    opt = torch.optim.Adam([q for q in p.parameters() if q.requires_grad], lr=2e-3)
    losses = []
    for _ in range(12):
        torch.manual_seed(7)                                              # same noise / timesteps every step
        loss = p(batch)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.8 * losses[0], losses
    act = p.predict_action(batch, steps=2)
    assert act.shape == (2, a.action_horizon, a.action_dim) and torch.isfinite(act).all()
    assert p.policy.last_losses


@pytest.mark.parametrize("name", ["dreamzero", "lingbot_va"])
def test_precomputed_feature_cache_matches_online_encoding(name, tmp_path):
    """Build -> validate -> train from the cache: the loss equals the loss with the codec / encoders in the loop; a stale
    or damaged cache is reported."""
    import json
    import os
    import numpy as np
    from loongforge_b200.embodied.data import PrecomputedFeatures, SyntheticEpisodes, build_dataset, collate
    from loongforge_b200.embodied.models import build_policy
    from tools.data_preprocess import embodied_precompute as E

    a = validate(EmbodiedArgs(model_name=name, model_overrides={"size": "tiny"}, image_size=32, action_horizon=4,
                              video_frames=9 if name == "dreamzero" else 5, output_dir=str(tmp_path / "run")))
    torch.manual_seed(a.seed)
    policy = build_policy(name, a)
    small = SyntheticEpisodes(a, num_episodes=1, episode_len=10)
    cache = str(tmp_path / "cache")
    m = E.build(a, cache, shard_size=4, batch_size=3, dtype="float32", policy=policy, dataset=small)
    assert m["complete"] and [s["count"] for s in m["shards"]] == [4, 4, 2] and "latents" in m["arrays"] and "text_emb" in m["arrays"]
    assert ("image_tokens" in m["arrays"]) == (name == "dreamzero")
    assert E.validate(cache, deep=True, expected_fingerprint=E.fingerprint(policy, a)) == []
    ds = PrecomputedFeatures(small, cache)
    assert "video" not in ds[5] and ds[5]["latents"].shape == tuple(m["arrays"]["latents"]["shape"])
    batch_cached, batch_raw = collate([ds[i] for i in (3, 4)]), collate([small[i] for i in (3, 4)])
    torch.manual_seed(11)
    l_cached = policy(batch_cached)
    torch.manual_seed(11)
    l_raw = policy(batch_raw)
    assert abs(float(l_cached) - float(l_raw)) < 1e-5 * max(1.0, abs(float(l_raw)))
    # resume: a build over the finished cache does nothing and keeps the manifest
    before = os.path.getmtime(os.path.join(cache, "features_00001.npz"))
    E.build(a, cache, shard_size=4, batch_size=3, dtype="float32", policy=policy, dataset=small)
    assert os.path.getmtime(os.path.join(cache, "features_00001.npz")) == before
    # other frozen weights -> another fingerprint; a missing shard and a wrong shape are found
    with torch.no_grad():
        next(policy.policy.vae.parameters()).add_(1.0)
    assert any("fingerprint" in p for p in E.validate(cache, expected_fingerprint=E.fingerprint(policy, a)))
    os.remove(os.path.join(cache, "features_00002.npz"))
    assert any("features_00002.npz is missing" in p for p in E.validate(cache))
    with np.load(os.path.join(cache, "features_00000.npz")) as z:
        arrays = {k: z[k] for k in z.files}
    arrays["latents"] = arrays["latents"][:, :, :1]
    np.savez(os.path.join(cache, "features_00000.npz"), **arrays)
    assert any("latents has shape" in p for p in E.validate(cache))
    with pytest.raises(ValueError):
        PrecomputedFeatures(SyntheticEpisodes(a, num_episodes=2, episode_len=10), cache)


def _wm_dist(rank, world, name, strategy, out):
    from loongforge_b200.embodied.distributed import DistContext
    from loongforge_b200.embodied.trainer import build_trainer

    ctx = DistContext()
    ctx.rank, ctx.world, ctx.local_rank = rank, world, rank
    a = validate(EmbodiedArgs(model_name=name, model_overrides={"size": "tiny"}, image_size=32, action_horizon=4,
                              video_frames=9 if name == "dreamzero" else 0 if name.startswith(("groot", "xvla")) else 5, train_steps=2, per_device_batch_size=2, output_dir=out,
                              strategy=strategy, fsdp_wrap_patterns=["auto"], fsdp_min_num_params=5000, fsdp_leftover_min_num_params=20000,
                              hsdp_shard_size=2 if strategy == "hsdp" else None, log_interval=1))
    t = build_trainer(a, ctx)
    m = t.train()
    full = sum(float(p.full_tensor().float().sum()) if hasattr(p, "full_tensor") else float(p.float().sum()) for p in t.model.parameters())
    return m["loss"], full


@pytest.mark.parametrize("name,strategy,world", [("lingbot_va", "fsdp", 2), ("fastwam", "fsdp", 2), ("dreamzero", "fsdp", 2),
                                                 ("cosmos3", "fsdp", 2), ("dreamzero", "zero1", 2), ("lingbot_va", "hsdp", 4),
                                                 ("groot_n1_6", "fsdp", 2), ("groot_n1_7", "fsdp", 2), ("xvla", "fsdp", 2)])
def test_world_models_train_sharded(name, strategy, world, tmp_path):
    """The automatic FSDP plan (and ZeRO-1 / HSDP) on the world-model policies: two steps on gloo ranks, finite loss, equal
    weights on all ranks — the policies that run joint attention over several experts name their no-wrap classes."""
    import math
    from tests.dist_utils import run_distributed

    res = run_distributed(_wm_dist, world, name, strategy, str(tmp_path))
    assert all(math.isfinite(r[0]) for r in res)
    assert max(abs(r[1] - res[0][1]) for r in res) < 1e-3 * max(1.0, abs(res[0][1]))


@pytest.mark.parametrize("name", ["lingbot_va", "fastwam", "dreamzero", "cosmos3", "pi05", "groot_n1_6", "groot_n1_7", "xvla"])
def test_policies_run_in_bf16(name):
    """`bf16: true` casts the whole policy (codec and towers included) and the floating-point inputs: loss, gradients and
    sampled actions stay finite."""
    from loongforge_b200.embodied.data import SyntheticEpisodes, collate
    from loongforge_b200.embodied.models import build_policy

    world = name in ("lingbot_va", "fastwam", "dreamzero", "cosmos3")
    a = validate(EmbodiedArgs(model_name=name, model_overrides={"size": "tiny"}, image_size=32, action_horizon=4,
                              video_frames=(9 if name == "dreamzero" else 5) if world else 0))
    torch.manual_seed(0)
    p = build_policy(name, a).to(torch.bfloat16)
    b = collate([SyntheticEpisodes(a)[i] for i in range(2)])
    b = {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in b.items()}
    loss = p(b)
    loss.backward()
    assert torch.isfinite(loss.detach().float())
    grads = [q.grad for q in p.parameters() if q.grad is not None]
    assert grads and all(torch.isfinite(g.float()).all() for g in grads)
    act = p.predict_action(b, steps=2)
    assert act.shape == (2, 4, a.action_dim) and torch.isfinite(act.float()).all()


def test_segment_attention_equals_dense_mask():
    """Block-constant masks in run form: same mask, same attention output (grouped-query heads included)."""
    from loongforge_b200.embodied.dreamzero import block_causal_mask
    from loongforge_b200.embodied.fastwam import mot_mask, mot_segment_mask
    from loongforge_b200.embodied.lingbot_va import teacher_forcing_mask
    from loongforge_b200.embodied.wan_blocks import SegmentMask, contiguous_runs, masked_attention

    torch.manual_seed(0)
    order = torch.tensor([0, 0, 0, 2, 2, 2, 1, 1, 3, 3, 0, 0, 0, 2, 2, 2, 1, 1, 3, 3])
    noisy = torch.tensor([1] * 10 + [0] * 10, dtype=torch.bool)
    st, en, rep = contiguous_runs(order, noisy.long())
    assert st == [0, 3, 6, 8, 10, 13, 16, 18] and en[-1] == 20
    cases = [(SegmentMask(st, en, teacher_forcing_mask(order[rep], noisy[rep], 2)), teacher_forcing_mask(order, noisy, 2))]
    for tf in (True, False):
        for off in (0, 1):
            a = (5, 3, 2, 4, 2, 2, 1, tf, 1 if tf else -1, None, off)
            cases.append((block_causal_mask(*a, segments=True), block_causal_mask(*a)))
    for variant, mode in (("fastwam", "first_frame_causal"), ("joint", "per_frame_causal"), ("idm", "bidirectional"),
                          ("idm", "per_frame_causal")):
        cases.append((mot_segment_mask(variant, 3, 4, 5, mode), mot_mask(variant, 3, 4, 5, mode)))
    from loongforge_b200.embodied.cosmos3 import pack_samples, packed_attention_mask, packed_segment_mask
    seq = pack_samples([torch.arange(1, 6), torch.arange(1, 4)], [(3, 2, 2), (2, 2, 2)], [4, 2])
    for tc in (True, False):
        cases.append((packed_segment_mask(seq, tc), packed_attention_mask(seq, tc)))
    for seg, dense in cases:
        assert isinstance(seg, SegmentMask) and torch.equal(seg.dense(), dense)
        L = dense.shape[0]
        q, k, v = torch.randn(2, L, 4, 8), torch.randn(2, L, 2, 8), torch.randn(2, L, 2, 8)
        assert torch.allclose(masked_attention(q, k, v, seg), masked_attention(q, k, v, dense), atol=1e-5)
    q = torch.randn(1, 20, 2, 8, requires_grad=True)
    masked_attention(q, q, q, cases[0][0]).sum().backward()
    g = q.grad.clone()
    q.grad = None
    masked_attention(q, q, q, cases[0][1]).sum().backward()
    assert torch.allclose(g, q.grad, atol=1e-5)


@pytest.mark.parametrize("name", ["lingbot_va", "fastwam", "dreamzero", "cosmos3"])
def test_policies_give_the_same_loss_with_segment_attention(name):
    import importlib
    mod = importlib.import_module(f"loongforge_b200.embodied.{name}")
    cfg_cls = {"lingbot_va": "LingBotVAConfig", "fastwam": "FastWAMConfig", "dreamzero": "DreamZeroConfig",
               "cosmos3": "Cosmos3Config"}[name]
    pol_cls = {"lingbot_va": "LingBotVAPolicy", "fastwam": "FastWAMPolicy", "dreamzero": "DreamZeroPolicy",
               "cosmos3": "Cosmos3Policy"}[name]
    losses = []
    for seg in (True, False):
        torch.manual_seed(0)
        p = getattr(mod, pol_cls)(getattr(mod, cfg_cls).tiny(action_dim=7, segment_attention=seg))
        torch.manual_seed(1)
        losses.append(float(p(_batch())))
    assert abs(losses[0] - losses[1]) < 1e-5 * max(1.0, abs(losses[1])), losses
