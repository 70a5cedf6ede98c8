"""Weight files: the one error that lists everything, alternative names, dtypes (no device)."""
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import transformer_b200 as tb
from transformer_b200.architectures.llama import tensor_plan
from transformer_b200.config import LlamaMeta
from transformer_b200.weights import WeightError, load_weights
from tiny import TINY_A, TINY_B, TINY_DENSE, make_folder

CPU = torch.device("cpu")


def _rules(cfg):
    return tensor_plan(LlamaMeta.from_dict(cfg))


def test_random_folder_loads_and_keeps_types(tmp_path):
    folder = make_folder(tmp_path, "A")
    files = load_file(os.path.join(folder, "model.safetensors"))
    assert files["blk.0.attn_qkv.weight"].dtype == torch.bfloat16
    assert files["output_norm.weight"].dtype == torch.float32        # a 32-bit tensor stays 32-bit
    assert torch.all(files["blk.1.ffn_norm.weight"] == 1)
    w = load_weights(folder, _rules(TINY_A), torch.bfloat16, CPU)
    assert w[("layers", 0, "mixer", "wqkv")].dtype == torch.bfloat16
    assert w[("final_norm", "weight")].dtype == torch.float32
    w32 = load_weights(folder, _rules(TINY_A), torch.float32, CPU)
    assert w32[("layers", 0, "mixer", "wqkv")].dtype == torch.float32
    assert torch.equal(w32[("layers", 0, "mixer", "wqkv")], w[("layers", 0, "mixer", "wqkv")].float())


def test_same_seed_same_folder(tmp_path):
    a = tb.write_random_model(str(tmp_path / "a"), TINY_A, seed=7)
    b = tb.write_random_model(str(tmp_path / "b"), TINY_A, seed=7)
    c = tb.write_random_model(str(tmp_path / "c"), TINY_A, seed=8)
    fa, fb, fc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(torch.equal(fa[k], fb[k]) for k in fa)
    assert not torch.equal(fa["token_embd.weight"], fc["token_embd.weight"])


def test_tied_head_shares_the_embedding(tmp_path):
    folder = make_folder(tmp_path, "B")
    assert "output.weight" not in load_file(os.path.join(folder, "model.safetensors"))
    w = load_weights(folder, _rules(TINY_B), torch.float32, CPU)
    assert w[("head", "weight")] is w[("embedding", "table")]


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    folder = make_folder(tmp_path, "A")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["blk.1.ffn_norm.weight"]
    del t["output.weight"]
    t["blk.0.attn_output.weight"] = t["blk.0.attn_output.weight"][:, :-1].contiguous()
    t["blk.7.extra.weight"] = torch.zeros(3)
    t["token_embd.weight"] = t["token_embd.weight"].to(torch.int32)
    bad = str(tmp_path / "bad")
    os.makedirs(bad)
    save_file(t, os.path.join(bad, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(bad, _rules(TINY_A), torch.bfloat16, CPU)
    err = e.value
    assert set(err.missing) == {"blk.1.ffn_norm.weight", "output.weight"}
    assert err.unexpected == ["blk.7.extra.weight"]
    assert [n for n, *_ in err.wrong_shape] == ["blk.0.attn_output.weight"]
    assert [n for n, *_ in err.wrong_type] == ["token_embd.weight"]
    msg = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "blk.7.extra.weight", "[64, 63]", "[64, 64]"):
        assert word in msg


def test_separate_q_k_v_and_gate_up_are_merged(tmp_path):
    folder = make_folder(tmp_path, "A")
    t = load_file(os.path.join(folder, "model.safetensors"))
    m = LlamaMeta.from_dict(TINY_A)
    q, kv = m.nh * m.dh, m.nkvh * m.dh
    split = dict(t)
    for i in range(m.nblk):
        w = split.pop(f"blk.{i}.attn_qkv.weight")
        split[f"blk.{i}.attn_q.weight"] = w[:q].contiguous()
        split[f"blk.{i}.attn_k.weight"] = w[q:q + kv].contiguous()
        split[f"blk.{i}.attn_v.weight"] = w[q + kv:].contiguous()
        gu = split.pop(f"blk.{i}.ffn_gate_up_exps.weight")
        split[f"blk.{i}.ffn_gate_exps.weight"] = gu[:, :m.di].contiguous()
        split[f"blk.{i}.ffn_up_exps.weight"] = gu[:, m.di:].contiguous()
    d2 = str(tmp_path / "split")
    os.makedirs(d2)
    save_file(split, os.path.join(d2, "model.safetensors"))
    a = load_weights(folder, _rules(TINY_A), torch.bfloat16, CPU)
    b = load_weights(d2, _rules(TINY_A), torch.bfloat16, CPU)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    # a half-present alternative is reported by what it lacks
    del split["blk.0.attn_k.weight"]
    d3 = str(tmp_path / "split_bad")
    os.makedirs(d3)
    save_file(split, os.path.join(d3, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(d3, _rules(TINY_A), torch.bfloat16, CPU)
    assert e.value.missing == ["blk.0.attn_k.weight"] and not e.value.unexpected


def test_one_matrix_per_expert_is_stacked(tmp_path):
    folder = make_folder(tmp_path, "A")
    t = load_file(os.path.join(folder, "model.safetensors"))
    m = LlamaMeta.from_dict(TINY_A)
    per = dict(t)
    for i in range(m.nblk):
        gu = per.pop(f"blk.{i}.ffn_gate_up_exps.weight")
        dn = per.pop(f"blk.{i}.ffn_down_exps.weight")
        for e in range(m.nexp):
            per[f"blk.{i}.ffn_gate.{e}.weight"] = gu[e, :m.di].contiguous()
            per[f"blk.{i}.ffn_up.{e}.weight"] = gu[e, m.di:].contiguous()
            per[f"blk.{i}.ffn_down.{e}.weight"] = dn[e].contiguous()
    d2 = str(tmp_path / "per_expert")
    os.makedirs(d2)
    save_file(per, os.path.join(d2, "model.safetensors"))
    a = load_weights(folder, _rules(TINY_A), torch.bfloat16, CPU)
    b = load_weights(d2, _rules(TINY_A), torch.bfloat16, CPU)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    del per["blk.1.ffn_up.2.weight"]
    d3 = str(tmp_path / "per_expert_bad")
    os.makedirs(d3)
    save_file(per, os.path.join(d3, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(d3, _rules(TINY_A), torch.bfloat16, CPU)
    assert e.value.missing == ["blk.1.ffn_up.2.weight"] and not e.value.unexpected


def test_dense_plan_has_no_router(tmp_path):
    names = {n for r in _rules(TINY_DENSE) for n in r.canonical.names}
    assert "blk.0.ffn_gate_up.weight" in names and not any("gate_inp" in n or "exps" in n for n in names)


def test_missing_folder_and_file(tmp_path):
    with pytest.raises(FileNotFoundError):
        tb.read_config(str(tmp_path))
    with pytest.raises(FileNotFoundError):
        load_weights(str(tmp_path), _rules(TINY_A), torch.bfloat16, CPU)
