"""The vision-language trainer under tensor / pipeline parallelism and encoder heterogeneous data parallelism must
follow the single-process trajectory (same data, same seed)."""
import pytest

from dist_utils import run_distributed


_REF = {}


def _run(rank, world, dims_kw, vlm_kw, steps=2):
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator

    lm = get_model_config("tiny-llama", position_embedding_type="mrope", mrope_section=[8, 12, 12])
    if dims_kw.get("tp", 1) > 1:
        lm.sequence_parallel = True
    vit = get_model_config("tiny-vit")
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=128, train_iters=steps, lr=1e-3, clip_grad=1.0,
                     log_interval=1000)
    tr = VLMTrainer(lm, tc, ParallelDims(**dims_kw), vit_cfg=vit, images_per_sample=2, image_size=112, **vlm_kw)
    st = tr.st
    it = synthetic_vlm_iterator(lm.vocab_size, 128, images_per_sample=2, image_size=112, pin_memory=False,
                                dp_rank=st.dp_rank, dp_size=st.dp_size, seed=9)
    out = []
    for _ in range(steps):
        m = tr.train_step(it)
        out.append((m.get("lm loss"), m["grad_norm"]))
    return out


@pytest.mark.parametrize("dims,vlm_kw,world", [
    ({"tp": 2}, {}, 2),                                   # decoder TP 2 + SP, encoder TP 1 (replicated on both ranks)
    ({"tp": 2}, {"encoder_tp": 2}, 2),                    # encoder sharded like the decoder
    ({"tp": 2}, {"encoder_hetero_dp": True}, 2),          # each TP rank encodes a different micro-batch
    ({"pp": 2}, {}, 2),                                   # encoder on the first stage only
    ({}, {}, 2),                                          # data parallel
    ({"tp": 2}, {"full_hetero_dp": True}, 2),             # encoder data parallel over the TP group, ahead of the step
    ({"pp": 2}, {"full_hetero_dp": True}, 2),             # ... over the pipeline stages (replica on the last stage)
    ({"tp": 2, "pp": 2}, {"full_hetero_dp": True, "full_hetero_cpu_offload": True}, 4),
])
def test_vlm_layouts_match_single_process(dims, vlm_kw, world):
    if "ref" not in _REF:
        _REF["ref"] = run_distributed(_run, 1, {}, {})[0]
    ref = _REF["ref"]
    res = run_distributed(_run, world, dict(dims), dict(vlm_kw))
    got = [r for r in res if r[0][0] is not None][-1]
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 2e-4 * abs(l0) and abs(g0 - g1) < 1e-3 * max(1, g0), (ref, got)
    for r in res:  # every rank reports the same global gradient norm
        assert all(abs(a[1] - b[1]) < 1e-5 * max(1, b[1]) for a, b in zip(r, got)), res


def _ckpt_worker(rank, world, tmp, dims_kw, vlm_kw, mode):
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator

    lm = get_model_config("tiny-llama", position_embedding_type="mrope", mrope_section=[8, 12, 12])
    if dims_kw.get("tp", 1) > 1:
        lm.sequence_parallel = True
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=128, train_iters=4, lr=1e-3, clip_grad=1.0,
                     log_interval=1000)
    tr = VLMTrainer(lm, tc, ParallelDims(**dims_kw), vit_cfg=get_model_config("tiny-vit"), images_per_sample=2,
                    image_size=112, **vlm_kw)
    st = tr.st
    it = synthetic_vlm_iterator(lm.vocab_size, 128, images_per_sample=2, image_size=112, pin_memory=False,
                                dp_rank=st.dp_rank, dp_size=st.dp_size, seed=9)
    if mode == "save":
        for _ in range(2):
            tr.train_step(it)
        tr.save_checkpoint(tmp)
    else:
        assert tr.load_checkpoint(tmp) == 2
        for _ in range(2 * 4 // st.dp_size):
            next(it)
    m = tr.train_step(it)
    return m.get("lm loss"), m["grad_norm"]


@pytest.mark.parametrize("save,load", [
    (({"tp": 2}, {}, 2), ({"pp": 2}, {}, 2)),                                   # encoder TP 1 beside decoder TP 2
    (({"tp": 2}, {"encoder_tp": 2}, 2), ({}, {}, 1)),
    (({"pp": 2}, {"full_hetero_dp": True}, 2), ({"tp": 2}, {"encoder_hetero_dp": True}, 2)),  # encoder replica not saved
])
def test_vlm_checkpoints_reshard(save, load, tmp_path):
    a = run_distributed(_ckpt_worker, save[2], str(tmp_path), save[0], save[1], "save")
    b = run_distributed(_ckpt_worker, load[2], str(tmp_path), load[0], load[1], "load")
    ga = [x for x in a if x[0] is not None][-1]
    gb = [x for x in b if x[0] is not None][-1]
    assert abs(ga[0] - gb[0]) < 1e-4 * abs(ga[0]) and abs(ga[1] - gb[1]) < 1e-3 * max(1, ga[1]), (ga, gb)


def _hf_worker(rank, world, tmp, dims_kw, vlm_kw, mode):
    import os

    from loongforge_b200.ckpt.hf_bridge import load_hf_checkpoint_online, save_hf_checkpoint
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.trainer import TrainConfig
    from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator

    lm = get_model_config("tiny-llama", add_qkv_bias=True, position_embedding_type="mrope", mrope_section=[8, 12, 12])
    if dims_kw.get("tp", 1) > 1:
        lm.sequence_parallel = True
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=128, train_iters=4, lr=1e-3, clip_grad=1.0,
                     log_interval=1000)
    tr = VLMTrainer(lm, tc, ParallelDims(**dims_kw), vit_cfg=get_model_config("tiny-vit"), images_per_sample=2,
                    image_size=112, **vlm_kw)
    st = tr.st
    it = synthetic_vlm_iterator(lm.vocab_size, 128, images_per_sample=2, image_size=112, pin_memory=False,
                                dp_rank=st.dp_rank, dp_size=st.dp_size, seed=9)
    if mode == "save":
        for _ in range(2):
            tr.train_step(it)
        save_hf_checkpoint(tr, os.path.join(tmp, "hf"), family="qwen2_5_vl")
    else:
        load_hf_checkpoint_online(tr, os.path.join(tmp, "hf"), family="qwen2_5_vl")
        for _ in range(2 * 4 // st.dp_size):
            next(it)
    m = tr.train_step(it)
    return m.get("lm loss"), m["grad_norm"]


def test_vlm_hugging_face_export_and_online_load_across_layouts(tmp_path):
    """Trained VLM (decoder TP 2, encoder TP 1) -> Hugging Face Qwen2.5-VL layout -> loaded online under PP 2 and
    under TP 2 with the encoder sharded as well: the next step is the one the exporting run takes."""
    import os

    a = run_distributed(_hf_worker, 2, str(tmp_path), {"tp": 2}, {}, "save")
    assert os.path.isfile(tmp_path / "hf" / "config.json")
    ga = [x for x in a if x[0] is not None][-1]
    for dims, kw in (({"pp": 2}, {}), ({"tp": 2}, {"encoder_tp": 2})):
        b = run_distributed(_hf_worker, 2, str(tmp_path), dims, kw, "load")
        gb = [x for x in b if x[0] is not None][-1]
        assert abs(ga[0] - gb[0]) < 1e-4 * abs(ga[0]) and abs(ga[1] - gb[1]) < 1e-3 * max(1, ga[1]), (ga, gb)
    # export again from a run whose encoder is sharded too: the files must hold the same tensors
    import shutil

    from tools.convert_checkpoint.convert import load_hf
    first = load_hf(str(tmp_path / "hf"))
    shutil.rmtree(tmp_path / "hf")
    c = run_distributed(_hf_worker, 2, str(tmp_path), {"tp": 2}, {"encoder_tp": 2}, "save")
    second = load_hf(str(tmp_path / "hf"))
    assert set(first) == set(second)
    import torch
    worst = max(float((first[k].float() - second[k].float()).abs().max()) for k in first)
    assert worst < 2e-4, worst  # two independent training runs in different layouts: summation order differs


def _hetero_balance(rank, world):
    import torch

    from loongforge_b200.models.omni import ENCODER_STATE, OmniCombinationModel
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel import state as ps

    ps.initialize_model_parallel(ps.ParallelDims(tp=2))
    ps.create_parallel_state(ENCODER_STATE, ps.ParallelDims(tp=1))
    lm = get_model_config("tiny-llama")
    vit = get_model_config("tiny-vit")
    outs = {}
    for hetero in (False, True):
        model = OmniCombinationModel(lm, vit, image_token_id=lm.vocab_size - 1, encoder_hetero_dp=hetero)
        g = torch.Generator().manual_seed(0)
        grid = torch.tensor([[1, 8, 8], [1, 4, 4], [1, 4, 8], [1, 4, 4]])   # 64 + 16 + 32 + 16 patches
        pixels = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 14 * 14, generator=g)
        emb = model.encode_images(pixels, grid)
        emb.pow(2).sum().backward()
        gsum = model.encoder_model.image_projector.linear_fc2.weight.grad.clone()
        if hetero:
            torch.distributed.all_reduce(gsum)   # partial per rank under hetero-DP (the trainer sums them)
        outs[hetero] = (emb.detach(), gsum)
    return float((outs[True][0] - outs[False][0]).abs().max()), float((outs[True][1] - outs[False][1]).abs().max())


def test_encoder_hetero_dp_balances_images_by_patches():
    """Four images of 64 / 16 / 32 / 16 patches over two ranks: 64 on one rank, 16 + 32 + 16 on the other; the
    embeddings come back in image order and the encoder gradients add up to the unsplit ones."""
    for err_emb, err_grad in run_distributed(_hetero_balance, 2):
        assert err_emb < 1e-5 and err_grad < 1e-3, (err_emb, err_grad)
