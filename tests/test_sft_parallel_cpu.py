"""Packed-sequence fine-tuning (several sequences per row, loss on a subset of tokens, optional LoRA adapters) must
give the same trajectory under tensor / pipeline / context / expert parallelism as in one process."""
import pytest
import torch

from dist_utils import run_distributed


_REF = {}


def _run(rank, world, model_name, dims_kw, lora):
    from loongforge_b200.models.registry import get_model_config
    from loongforge_b200.parallel.state import ParallelDims
    from loongforge_b200.runtime.sft import SFTTrainer
    from loongforge_b200.runtime.trainer import TrainConfig

    cfg = get_model_config(model_name)
    if dims_kw.get("tp", 1) > 1:
        cfg.sequence_parallel = True
    tc = TrainConfig(micro_batch_size=1, global_batch_size=4, seq_length=64, train_iters=2, lr=1e-3, clip_grad=1.0,
                     log_interval=1000, training_phase="sft")
    tr = SFTTrainer(cfg, tc, ParallelDims(**dims_kw), lora=dict(rank=4, alpha=8) if lora else None)
    st = tr.st

    def rows():
        g = torch.Generator().manual_seed(5)
        i = 0
        while True:
            lens = [[20, 28, 16], [32, 32], [8, 40, 16], [64]][i % 4]   # sequence lengths need not divide by 2 * cp
            tok = torch.randint(0, cfg.vocab_size, (1, 65), generator=g)
            mask = (torch.rand(1, 64, generator=g) > 0.4).float()
            cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
            b = {"tokens": tok[:, :-1], "labels": tok[:, 1:], "loss_mask": mask, "cu_seqlens": cu,
                 "position_ids": torch.cat([torch.arange(n) for n in lens])[None], "num_valid_tokens": int(mask.sum())}
            if i % st.dp_size == st.dp_rank:
                yield b
            i += 1

    it = rows()
    return [(m.get("lm loss"), m["grad_norm"]) for m in (tr.train_step(it) for _ in range(2))]


@pytest.mark.parametrize("model,dims,lora,world", [
    ("tiny-llama", {"tp": 2}, False, 2),
    ("tiny-llama", {"cp": 2}, False, 2),
    ("tiny-llama", {"tp": 2}, True, 2),
    ("tiny-llama", {"pp": 2}, True, 2),
    ("tiny-qwen3-moe", {"tp": 2, "ep": 2}, True, 4),
    ("tiny-deepseek", {"cp": 2}, False, 2),
])
def test_packed_sft_matches_single_process(model, dims, lora, world):
    if (model, lora) not in _REF:
        _REF[(model, lora)] = run_distributed(_run, 1, model, {}, lora)[0]
    ref = _REF[(model, lora)]
    res = run_distributed(_run, world, model, dict(dims), lora)
    got = [r for r in res if r[0][0] is not None][-1]
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) < 2e-4 * abs(l0) and abs(g0 - g1) < 5e-4 * max(1, g0), (ref, got)
