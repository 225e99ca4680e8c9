"""Checkpoint-format and dump tools: the DeepSeek-V4 layouts (published fp4 experts with power-of-two scales <-> fp8
serving layout <-> bf16) on a miniature checkpoint written by the test, and the per-token dump alignment / comparison."""
import json
import os
import subprocess
import sys

import pytest
import torch

from gcore_b200.tools import dsv4_ckpt as T

E8 = getattr(torch, "float8_e8m0fnu", None)
pytestmark = pytest.mark.skipif(E8 is None, reason="this torch has no e8m0 dtype")


def _published(tmp, seed=0):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    os.makedirs(tmp, exist_ok=True)

    def fp4(rows, cols):
        x = torch.randn(rows, cols, generator=g) * torch.exp2(torch.randint(-3, 3, (rows, 1), generator=g).float())
        blk = x.view(rows, cols // 32, 32)
        s = torch.exp2(torch.ceil(torch.log2(blk.abs().amax(-1).clamp_min(2.0 ** -126) / 6.0)))
        return T.pack_fp4((blk / s[..., None]).view(rows, cols)), T.f32_to_e8m0(s)[0]

    def fp8(rows, cols):
        return T.bf16_to_fp8((torch.randn(rows, cols, generator=g) * 0.05).bfloat16())

    s0, s1 = {}, {}
    for e in range(2):
        for w, (r, c) in (("w1", (256, 128)), ("w2", (128, 256)), ("w3", (256, 128))):
            s0[f"layers.0.ffn.experts.{e}.{w}.weight"], s0[f"layers.0.ffn.experts.{e}.{w}.scale"] = fp4(r, c)
    s0["layers.0.ffn.shared_experts.w1.weight"], s0["layers.0.ffn.shared_experts.w1.scale"] = fp8(256, 128)
    s1["layers.0.attn.wo_a.weight"], s1["layers.0.attn.wo_a.scale"] = fp8(128, 256)
    s1["layers.0.attn.wq_a.weight"], s1["layers.0.attn.wq_a.scale"] = fp8(256, 128)
    s1["embed.weight"] = torch.randn(64, 128, generator=g).bfloat16()
    s1["layers.0.attn_norm.weight"] = torch.ones(128, dtype=torch.bfloat16)
    save_file(s0, os.path.join(tmp, "model-00001-of-00002.safetensors"))
    save_file(s1, os.path.join(tmp, "model-00002-of-00002.safetensors"))
    json.dump({"model_type": "deepseek_v4", "expert_dtype": "fp4"}, open(os.path.join(tmp, "config.json"), "w"))
    open(os.path.join(tmp, "tokenizer.json"), "w").write("{}")
    return {**s0, **s1}


def test_scalar_formats_round_trip():
    codes = torch.arange(256, dtype=torch.uint8)
    packed = codes.view(16, 16).view(torch.int8)
    v = T.unpack_fp4(packed)
    assert v.shape == (16, 32) and set(v.abs().unique().tolist()) == {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}
    assert torch.equal(T.pack_fp4(v).view(torch.uint8), packed.view(torch.uint8))   # every code, both signs of zero
    # ties go to the even mantissa: 0.25 -> 0, 0.75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4
    ties = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0]])
    assert T.unpack_fp4(T.pack_fp4(ties.clamp(max=6.0))).tolist() == [[0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0]]
    s = torch.tensor([1.0, 0.5, 3.0, 2.0 ** -20])
    c, inexact = T.f32_to_e8m0(s)
    assert inexact == 1 and T.e8m0_to_f32(c).tolist() == [1.0, 0.5, 4.0, 2.0 ** -20]


def test_published_to_fp8_and_back_is_exact(tmp_path):
    pub, fp8, back, bf = (str(tmp_path / n) for n in ("pub", "fp8", "back", "bf16"))
    orig = _published(pub)
    st = T.convert_dir(pub, fp8, "published2fp8")
    assert st.get("inexact_elements", 0) == 0
    from safetensors.torch import load_file
    a = load_file(os.path.join(fp8, "model-00001-of-00002.safetensors"))
    b = load_file(os.path.join(fp8, "model-00002-of-00002.safetensors"))
    w = a["layers.0.ffn.experts.1.w2.weight"]
    assert w.dtype == torch.float8_e4m3fn and w.shape == (128, 256)
    assert a["layers.0.ffn.experts.1.w2.scale"].dtype == torch.float32
    assert a["layers.0.ffn.experts.1.w2.scale"].shape == (1, 2)
    assert b["layers.0.attn.wo_a.weight"].dtype == torch.bfloat16 and "layers.0.attn.wo_a.scale" not in b
    assert b["layers.0.attn.wq_a.scale"].dtype == torch.float32
    assert torch.equal(b["layers.0.attn.wq_a.weight"].view(torch.uint8),
                       orig["layers.0.attn.wq_a.weight"].view(torch.uint8))            # dense bytes untouched
    assert "expert_dtype" not in json.load(open(os.path.join(fp8, "config.json")))
    assert os.path.exists(os.path.join(fp8, "tokenizer.json"))
    idx = json.load(open(os.path.join(fp8, "model.safetensors.index.json")))
    assert set(idx["weight_map"]) == set(a) | set(b)
    assert idx["metadata"]["total_size"] == sum(v.numel() * v.element_size() for v in list(a.values()) + list(b.values()))
    assert T.compare_dirs(pub, fp8)["equal"]                                              # same values, other codes

    T.convert_dir(fp8, back, "fp82published")
    rep = T.compare_dirs(pub, back)
    assert rep["equal"] and rep["compared"] == 11, rep
    c = {**load_file(os.path.join(back, "model-00001-of-00002.safetensors")),
         **load_file(os.path.join(back, "model-00002-of-00002.safetensors"))}
    assert set(c) == set(orig) and all(c[k].dtype == orig[k].dtype and c[k].shape == orig[k].shape for k in orig)
    assert json.load(open(os.path.join(back, "config.json")))["expert_dtype"] == "fp4"

    T.convert_dir(pub, bf, "to_bf16")
    d = {**load_file(os.path.join(bf, "model-00001-of-00002.safetensors")),
         **load_file(os.path.join(bf, "model-00002-of-00002.safetensors"))}
    assert not any(k.endswith(".scale") for k in d) and all(v.dtype == torch.bfloat16 for v in d.values())
    assert torch.equal(d["layers.0.ffn.experts.0.w1.weight"].float(),
                       T.fp4_dequant(orig["layers.0.ffn.experts.0.w1.weight"], orig["layers.0.ffn.experts.0.w1.scale"]))
    assert T.compare_dirs(pub, bf)["equal"]


def test_wide_scale_span_is_counted_and_difference_is_reported(tmp_path):
    # 1x32 scales 2^-12 and 2^0 inside one 128-block: the small block falls below e4m3's subnormals
    vals = torch.full((128, 128), 0.5)
    packed = T.pack_fp4(vals)
    s = torch.ones(128, 4)
    s[:, 0] = 2.0 ** -12
    q, s128, bad = T.fp4_to_fp8(packed, T.f32_to_e8m0(s)[0])
    assert float(s128) == 1.0 and bad == 128 * 32
    pub, other = str(tmp_path / "a"), str(tmp_path / "b")
    _published(pub, seed=0)
    _published(other, seed=1)
    rep = T.compare_dirs(pub, other)
    assert not rep["equal"] and rep["different"] > 0 and rep["worst"] is not None


def test_two_ranks_split_the_shards_and_rank0_merges_the_index(tmp_path):
    pub, out = str(tmp_path / "pub"), str(tmp_path / "out")
    _published(pub)
    env = dict(os.environ, WORLD_SIZE="2")
    cmd = [sys.executable, "-m", "gcore_b200.tools.dsv4_ckpt", "convert", "--direction", "published2fp8", "--src", pub,
           "--dst", out]
    p1 = subprocess.Popen(cmd, env=dict(env, RANK="1"))
    p0 = subprocess.run(cmd, env=dict(env, RANK="0"), capture_output=True, text=True, timeout=240)
    assert p1.wait(timeout=240) == 0 and p0.returncode == 0, p0.stderr[-400:]
    idx = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    assert len(set(idx["weight_map"].values())) == 2 and not [f for f in os.listdir(out) if f.startswith(".index")]
    assert T.compare_dirs(pub, out)["equal"]


def test_token_dump_alignment_and_comparison(tmp_path):
    """The per-token dump tool: fields brought to the trainer's lengths; two dumps compared field by field."""
    from gcore_b200.tools import align_dumps as A
    row = {"prompt_length": 2, "group_id": 0, "reward": 1.0, "tokens": [5, 6, 7, 8, 9],
           "mask": [0, 1, 1, 1, 0], "logprobs": [0.0, -1.0, -2.0, -3.0, 0.0], "advantages": [0.0, 0.5, 0.5, 0.5, 0.0]}
    al = A.align_sample(row, pad_multiple=4)
    assert al["padded_seqlen"] == 8 and al["tokens"] == [5, 6, 7, 8, 9, 0, 0, 0]
    assert len(al["mask"]) == len(al["logprobs"]) == 7 and al["logprobs"][:4] == [0.0, -1.0, -2.0, -3.0]
    other = json.loads(json.dumps(row))
    other["logprobs"][2] = -2.25
    fa, fb = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    fa.write_text(json.dumps(row) + "\n" + json.dumps(row) + "\n")
    fb.write_text(json.dumps(row) + "\n" + json.dumps(other) + "\n")
    rep = A.compare_dumps(A.read_dump(str(fa)), A.read_dump(str(fb)))
    assert not rep["equal"] and rep["logprobs"]["first_difference"] == {"sample": 1, "position": 2, "a": -2.0, "b": -2.25}
    assert rep["logprobs"]["max_abs_diff"] == 0.25 and rep["advantages"]["first_difference"] is None
    assert A.compare_dumps(A.read_dump(str(fa)), A.read_dump(str(fa)))["equal"]
    assert A.main(["compare", "--a", str(fa), "--b", str(fb)]) == 1
