"""Family task encoders: token counts per medium, label masking, position ids, packing compatibility."""
import numpy as np
import pytest
import torch

from loongforge_b200.data import position_ids as P
from loongforge_b200.data import task_encoders as TE
from loongforge_b200.data.multimodal import OnlinePacker, VisionPreprocess

IMG, VID, VS, VE, EOS = 900, 901, 902, 903, 2


def _tok(text):
    return [10 + (ord(c) % 50) for c in text]


def _img(h, w, seed=0):
    return np.random.RandomState(seed).randint(0, 255, (h, w, 3), dtype=np.uint8)


def _sp(**kw):
    return TE.SpecialTokens(image=IMG, video=VID, vision_start=VS, vision_end=VE, eos=EOS, **kw)


def _vision():
    return VisionPreprocess(patch_size=14, temporal_patch_size=2, merge_size=2, min_pixels=28 * 28, max_pixels=28 * 28 * 64)


CHAT = {"images": [_img(56, 84)], "conversation": [{"role": "user", "content": "look <image> what?"},
                                                  {"role": "assistant", "content": "a cat"}]}


def test_qwen_encoder_counts_masks_and_positions():
    enc = TE.build_task_encoder("qwen2_vl", _tok, _sp(), _vision())
    out = enc.encode(CHAT)
    gh, gw = out["grid_thw"][0, 1:].tolist()
    n_img = (gh // 2) * (gw // 2)
    ids = out["tokens"].tolist()
    assert ids.count(IMG) == n_img and out["pixels"].shape == (gh * gw, 3 * 2 * 14 * 14)
    i0 = ids.index(VS)
    assert ids[i0 + 1] == IMG and ids[i0 + n_img + 1] == VE
    # loss only on the assistant turn (its text + eos), shifted by one; never on placeholders
    n_ans = len(_tok("a cat")) + 1
    assert int(out["loss_mask"].sum()) == n_ans
    assert out["loss_mask"][-n_ans - 1:-1].all() and out["loss_mask"][-1] == 0
    assert out["mrope"].shape == (3, len(ids))
    assert torch.equal(out["mrope"], P.mrope_ids(out["tokens"], out["grid_thw"], IMG, 2))
    # the three kinds of raw samples normalise to the same walker
    cap = enc.encode({"image": _img(56, 56), "caption": "a dog"})
    vqa = enc.encode({"image": _img(56, 56), "context": "what is it?", "answer": "a dog"})
    assert cap["tokens"].tolist().count(IMG) == vqa["tokens"].tolist().count(IMG) == 4


def test_video_encoding_families():
    frames = [_img(56, 56, s) for s in range(3)]  # padded to 4 frames = 2 temporal groups
    sample = {"videos": [frames], "conversation": [{"role": "user", "content": "<video> describe"},
                                                   {"role": "assistant", "content": "ok"}]}
    q2 = TE.build_task_encoder("qwen2_5_vl", _tok, _sp(), _vision(), fps=1.0, tokens_per_second=2.0).encode(sample)
    assert q2["video_grid_thw"].tolist() == [[2, 4, 4]] and q2["tokens"].tolist().count(VID) == 2 * 2 * 2
    assert q2["video_pixels"].shape == (2 * 16, 3 * 2 * 14 * 14)
    # second frame group sits second_per_grid_t * tokens_per_second = 2 * 2 = 4 steps later in the t stream
    t_pos = q2["mrope"][0][q2["tokens"] == VID]
    assert (t_pos[4:] - t_pos[:4]).unique().tolist() == [4]
    q3 = TE.build_task_encoder("qwen3_vl", _tok, _sp(), _vision(), fps=2.0).encode(sample)
    ids = q3["tokens"].tolist()
    assert ids.count(VID) == 8 and ids.count(VS) == 2  # one wrapped block per frame group, time stamps between
    kimi = TE.build_task_encoder("kimi_vl", _tok, _sp(), _vision()).encode(sample)
    assert kimi["tokens"].tolist().count(VID) == 2 * 2  # time pooled away
    mini = TE.build_task_encoder("minicpm_v", _tok, _sp(), _vision()).encode(sample)
    assert mini["tokens"].tolist().count(VID) == 2 * 1 * 1  # (4 / (2 * 2))^2 per group


def test_internvl_tiles_and_positions():
    enc = TE.build_task_encoder("internvl", _tok, _sp(), max_tiles=6, tokens_per_tile=16)
    out = enc.encode({"images": [_img(300, 900)], "conversation": [{"role": "user", "content": "<image> hi"},
                                                                   {"role": "assistant", "content": "yo"}]})
    n_tiles = out["pixel_tiles"].shape[0]
    assert n_tiles == 3 + 1 and out["pixel_tiles"].shape[1:] == (3, 448, 448)  # 3 x 1 grid + thumbnail
    assert out["tokens"].tolist().count(IMG) == n_tiles * 16
    pos = out["mrope"][0]
    inner = (out["tokens"] == IMG).nonzero().flatten()
    assert pos[inner[1]] == pos[inner[-1]]  # inner vision tokens share a position
    assert pos[-1] == pos.max() and (pos[1:] >= pos[:-1]).all()


def test_ernie_types_llava_wrappers_and_overlong_gating():
    ern = TE.build_task_encoder("ernie_vl", _tok, _sp(), _vision()).encode(CHAT)
    assert torch.equal(ern["token_type"], (ern["tokens"] == IMG).long())
    img_pos = ern["mrope"][:, ern["tokens"] == IMG]
    assert img_pos[0].unique().numel() == 1  # an image is one time step
    lla = TE.build_task_encoder("llava_ov", _tok, _sp(), _vision()).encode(CHAT)
    assert VS not in lla["tokens"].tolist()
    assert TE.build_task_encoder("qwen2_vl", _tok, _sp(), _vision(), max_length=8).encode(CHAT) is None
    long = {"images": [], "conversation": [{"role": "user", "content": "x" * 40}, {"role": "assistant", "content": "y" * 40}]}
    cut = TE.build_task_encoder("kimi_vl", _tok, _sp(), _vision(), max_length=50).encode(long)
    assert cut["tokens"].numel() == 50
    with pytest.raises(ValueError):
        TE.build_task_encoder("qwen2_vl", _tok, _sp(), _vision()).encode({"images": [], "conversation": CHAT["conversation"]})


def test_encoded_samples_pack():
    enc = TE.build_task_encoder("qwen3_vl", _tok, _sp(), _vision())
    packer = OnlinePacker(256, buffer_size=4, pad_to_seq_len=True)
    packs = []
    for s in range(5):
        packs += packer.add(enc.encode({"image": _img(56, 56 + 28 * (s % 2), s), "caption": "c" * (5 + s)}))
    packs += packer.flush()
    assert packs and all(p["tokens"].numel() == 256 and p["position_ids"].shape == (3, 256) for p in packs)
    assert sum(p["grid_thw"].shape[0] for p in packs) == 5


def test_position_id_registry():
    assert P.get_position_id_func("qwen3_vl") is P.qwen3_vl_ids
    with pytest.raises(KeyError):
        P.get_position_id_func("nope")


def test_video_members_of_shards_are_decoded_and_encoded(tmp_path):
    """An .mp4 next to the conversation in a shard -> frames sampled by --fps / --frame-num -> the <video> marker's
    placeholder tokens and video patches of the Qwen2.5-VL task encoder."""
    import json
    import cv2
    from loongforge_b200.data.multimodal import decode_video, webdataset_samples
    from loongforge_b200.data.task_encoders import build_task_encoder
    from tools.data_preprocess import vlm_to_webdataset as W

    src = tmp_path / "raw"
    src.mkdir()
    w = cv2.VideoWriter(str(src / "clip.mp4"), cv2.VideoWriter_fourcc(*"mp4v"), 10, (56, 56))
    for t in range(20):
        w.write(np.full((56, 56, 3), 10 * t, np.uint8))
    w.release()
    data = (src / "clip.mp4").read_bytes()
    assert len(decode_video(data)) == 20
    half = decode_video(data, fps=5)                                    # every second frame of a 10 fps clip
    assert len(half) == 10 and half[1].mean() > half[0].mean()
    four = decode_video(data, frame_num=4)
    assert len(four) == 4 and abs(float(four[-1].mean()) - 190) < 12     # first and last frame kept
    recs = [{"video": "clip.mp4", "conversations": [{"from": "human", "value": "<video> what happens?"}, {"from": "gpt", "value": "it brightens"}]}]
    W.write_shards(recs, str(tmp_path / "shards"), image_root=str(src))
    sample = next(webdataset_samples(str(tmp_path / "shards"), epochs=1, frame_num=4))
    assert len(sample["videos"]) == 1 and len(sample["videos"][0]) == 4 and sample["images"] == []
    enc = build_task_encoder("qwen2_5_vl", _tok, _sp(), _vision(), max_length=512)
    out = enc.encode(sample)
    assert "video_pixels" in out and out["video_grid_thw"][0][0] == 2    # 4 frames, temporal patch 2
    n_tok = int((out["tokens"] == enc.sp.video).sum()) if enc.sp.video is not None else int((out["tokens"] == enc.sp.image).sum())
    t, gh, gw = (int(x) for x in out["video_grid_thw"][0])
    assert n_tok == t * (gh // 2) * (gw // 2)


def test_videos_and_images_share_one_patch_stream_in_token_order():
    from loongforge_b200.data.multimodal import merge_video_into_image_stream, vlm_batch_iterator

    frames = [_img(56, 56, seed=s) for s in range(4)]
    sample = {"images": [_img(56, 84, seed=9), _img(28, 56, seed=8)], "videos": [frames],
              "conversation": [{"role": "user", "content": "first <image> then <video> and <image> ?"}, {"role": "assistant", "content": "ok"}]}
    enc_obj = TE.build_task_encoder("qwen2_5_vl", _tok, _sp(), _vision())
    enc = enc_obj.encode(sample)
    assert enc["media_order"].tolist() == [0, 1, 0]
    merged = merge_video_into_image_stream(enc, IMG, VID)
    g = merged["grid_thw"]
    assert g.shape == (3, 3) and torch.equal(g[0], enc["grid_thw"][0]) and torch.equal(g[1], enc["video_grid_thw"][0]) and torch.equal(g[2], enc["grid_thw"][1])
    assert merged["pixels"].shape[0] == int(g.prod(-1).sum()) and (merged["tokens"] == VID).sum() == 0
    n0, nv = int(g[0].prod()), int(g[1].prod())
    assert torch.equal(merged["pixels"][n0:n0 + nv].float(), enc["video_pixels"].float())        # the video sits between the images
    assert int((merged["tokens"] == IMG).sum()) == int((g.prod(-1) // 4).sum())                 # one placeholder per merged 2 x 2 patch
    assert torch.equal(merged["mrope"], enc["mrope"])                                             # positions come from the original ids
    batch = next(vlm_batch_iterator(iter([sample]), enc_obj, 512))
    assert batch["grid_thw"].shape == (3, 3) and batch["pixels"].shape[0] == int(batch["grid_thw"].prod(-1).sum())
