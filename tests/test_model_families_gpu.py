"""Every model family takes training steps on a GPU through the native kernels (bf16) and follows the fp32 CPU
trajectory of the same model, data and seed: dense Llama, Qwen3-MoE (router + grouped GEMM), DeepSeek MLA + DSA,
hybrid linear attention, MiniMax / MiMo (multi-token prediction), GLM, DeepSeek-V4 (compressed sparse attention +
hyper-connections), ERNIE multi-type MoE, the Qwen2.5-VL style vision-language model (windowed vision attention with
head dim 16 through the tcgen05 kernel) and the WAN diffusion transformer."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _steps(device, bf16, build, n=2):
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
    tr, it = build(device, bf16)
    out = []
    for _ in range(n):
        m = tr.train_step(it)
        out.append((m.get("lm loss", m.get("loss")), m["grad_norm"]))
    if device.type == "cuda":
        from loongforge_b200.ops import _ext

        torch.cuda.synchronize()
        _ext.check_status()
    ps.destroy_model_parallel()
    return out


def _compare(build, loss_tol=3e-2, norm_tol=0.15):
    ref = _steps(torch.device("cpu"), False, build)
    got = _steps(torch.device("cuda", 0), True, build)
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert l1 == l1 and abs(l0 - l1) < loss_tol * max(1.0, abs(l0)), (ref, got)
        assert abs(g0 - g1) < norm_tol * max(1.0, abs(g0)), (ref, got)


@pytest.mark.parametrize("name,ov", [
    ("tiny-llama", {}),
    ("tiny-qwen3-moe", {}),
    ("tiny-deepseek", {}),
    ("tiny-qwen3-next", {}),
    ("tiny-minimax", {}),
    ("tiny-mimo", {}),
    ("tiny-glm", {}),
    ("tiny-deepseek-v4", {}),
    ("tiny-ernie-vl", {}),
])
def test_llm_family_trains_on_gpu_like_on_cpu(name, ov):
    def build(device, bf16):
        from loongforge_b200.data.synthetic import synthetic_batch_iterator
        from loongforge_b200.models.registry import get_model_config
        from loongforge_b200.runtime.trainer import TrainConfig, Trainer

        cfg = get_model_config(name, **ov)
        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=2, lr=1e-3, clip_grad=1.0,
                         log_interval=1000, bf16=bf16, seed=21)
        tr = Trainer(cfg, tc, device=device)
        return tr, synthetic_batch_iterator(cfg.vocab_size, 256, 1, seed=3, pin_memory=False)

    _compare(build)


def test_vision_language_model_trains_on_gpu_like_on_cpu():
    def build(device, bf16):
        from loongforge_b200.models.registry import get_model_config
        from loongforge_b200.runtime.trainer import TrainConfig
        from loongforge_b200.runtime.vlm import VLMTrainer, synthetic_vlm_iterator

        lm = get_model_config("tiny-llama", position_embedding_type="mrope", mrope_section=[8, 12, 12])
        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=256, train_iters=2, lr=1e-3, clip_grad=1.0,
                         log_interval=1000, bf16=bf16, seed=22)
        tr = VLMTrainer(lm, tc, vit_cfg=get_model_config("tiny-vit"), images_per_sample=2, image_size=112,
                        device=device)
        return tr, synthetic_vlm_iterator(lm.vocab_size, 256, images_per_sample=2, image_size=112, pin_memory=False,
                                          seed=9)

    _compare(build)


@pytest.mark.parametrize("name", ["tiny-wan", "tiny-qwen-image"])
def test_diffusion_transformer_trains_on_gpu_like_on_cpu(name):
    def build(device, bf16):
        from loongforge_b200.runtime.diffusion_trainer import build_diffusion_trainer
        from loongforge_b200.runtime.trainer import TrainConfig

        tc = TrainConfig(micro_batch_size=1, global_batch_size=2, seq_length=64, train_iters=2, lr=1e-3, clip_grad=1.0,
                         log_interval=1000, bf16=bf16, seed=23)
        tr = build_diffusion_trainer(name, tc, device=device)
        return tr, tr.build_data_iterator(None)

    # the double-stream image model starts from losses below 1: allow bf16 noise of a few hundredths
    _compare(build, loss_tol=1e-1, norm_tol=0.25)
