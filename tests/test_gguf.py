"""The GGUF reader against files written by the ``gguf`` package (no device)."""

import numpy as np
import pytest
import torch

import transformer_b200 as tb
from transformer_b200.architectures.llama import tensor_plan
from transformer_b200.config import LlamaMeta, architecture_for
from transformer_b200.weights import WeightError, load_weights
from transformer_b200.weights.gguf import GGufError, GGufFile
from transformer_b200.weights.random_init import random_file_tensors
from tiny import TINY_A, TINY_B

gguf = pytest.importorskip("gguf")
CPU = torch.device("cpu")


def write_gguf(path, cfg, tensors, *, tokens=True, f16=(), quantize=None):
    m = LlamaMeta.from_dict(cfg)
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", m.nblk)
    w.add_uint32("llama.embedding_length", m.d)
    w.add_uint32("llama.attention.head_count", m.nh)
    w.add_uint32("llama.attention.head_count_kv", m.nkvh)
    w.add_uint32("llama.rope.dimension_count", m.dh)
    w.add_uint32("llama.feed_forward_length", m.di)
    w.add_uint32("llama.expert_count", m.nexp)
    w.add_uint32("llama.expert_used_count", m.nexp_use)
    w.add_uint32("llama.context_length", m.nctx)
    w.add_float32("llama.attention.layer_norm_rms_epsilon", m.epsilon)
    w.add_float32("llama.rope.freq_base", m.theta)
    w.add_string("rope_pairing", m.rope_pairing)
    if tokens:
        w.add_array("tokenizer.ggml.tokens", [f"t{i}" for i in range(m.nvoc)])
    w.add_uint32("tokenizer.ggml.eos_token_id", 2)
    for name, t in tensors.items():
        if name == quantize:
            blocks = np.zeros((t.shape[0], t.shape[1] // 32 * 18), dtype=np.uint8)     # Q4_0: 18 bytes per 32 values
            w.add_tensor(name, blocks, raw_dtype=gguf.GGMLQuantizationType.Q4_0)
        elif t.dtype == torch.bfloat16 and name in f16:
            w.add_tensor(name, t.to(torch.float16).numpy())
        elif t.dtype == torch.bfloat16:
            w.add_tensor(name, t.view(torch.int16).numpy().view(np.uint16), raw_shape=t.shape,
                         raw_dtype=gguf.GGMLQuantizationType.BF16)
        else:
            w.add_tensor(name, t.numpy())
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B])
def test_metadata_and_tensors_round_trip(cfg, tmp_path):
    rules = tensor_plan(LlamaMeta.from_dict(cfg))
    tensors = random_file_tensors(rules, seed=1, matrix_dtype=torch.bfloat16, std=0.1)
    path = write_gguf(str(tmp_path / "m.gguf"), cfg, tensors, f16=("blk.0.attn_output.weight",))
    f = GGufFile(path)
    assert f.metadata["general.architecture"] == "llama" and f.metadata["llama.block_count"] == cfg["num_hidden_layers"]
    assert f.shape_dtype("blk.0.attn_output.weight")[1] == "F16" and f.shape_dtype("token_embd.weight")[1] == "BF16"
    assert f.shape_dtype("output_norm.weight") == ((cfg["hidden_size"],), "F32")
    conf = tb.read_config(path)
    assert architecture_for(conf).name == "llama"
    want = LlamaMeta.from_dict(cfg)
    got = LlamaMeta.from_dict(conf)
    assert (got.nvoc, got.eos, got.tied) == (want.nvoc, (2,), want.tied), "vocabulary from the token list, tied from the missing head"
    import dataclasses
    assert abs(got.epsilon / want.epsilon - 1) < 1e-6 and abs(got.theta / want.theta - 1) < 1e-6   # stored as float32
    same = dict(eos=(), epsilon=0.0, theta=0.0)
    assert dataclasses.replace(got, **same) == dataclasses.replace(want, **same)
    loaded = load_weights(path, tensor_plan(got), torch.float32, CPU)
    for rule in rules:
        if rule.shared_with is None:
            ref = tensors[rule.canonical.names[0]].float()
            if rule.canonical.names[0] == "blk.0.attn_output.weight":
                ref = tensors[rule.canonical.names[0]].to(torch.float16).float()
            assert torch.equal(loaded[rule.dest], ref), rule.dest
    if want.tied:
        assert loaded[("head", "weight")] is loaded[("embedding", "table")]


def test_vocabulary_from_the_embedding_when_there_is_no_token_list(tmp_path):
    rules = tensor_plan(LlamaMeta.from_dict(TINY_A))
    tensors = random_file_tensors(rules, 1, torch.bfloat16)
    path = write_gguf(str(tmp_path / "m.gguf"), TINY_A, tensors, tokens=False)
    assert LlamaMeta.from_dict(tb.read_config(path)).nvoc == TINY_A["vocab_size"]


def test_quantized_tensors_are_named_in_the_error(tmp_path):
    rules = tensor_plan(LlamaMeta.from_dict(TINY_A))
    tensors = random_file_tensors(rules, 1, torch.bfloat16)
    path = write_gguf(str(tmp_path / "q.gguf"), TINY_A, tensors, quantize="blk.1.attn_qkv.weight")
    with pytest.raises(WeightError) as e:
        load_weights(path, rules, torch.bfloat16, CPU)
    assert [(n, t) for n, t, _ in e.value.wrong_type] == [("blk.1.attn_qkv.weight", "Q4_0")]


def test_broken_files(tmp_path):
    rules = tensor_plan(LlamaMeta.from_dict(TINY_A))
    tensors = random_file_tensors(rules, 1, torch.bfloat16)
    good = write_gguf(str(tmp_path / "g.gguf"), TINY_A, tensors)
    data = open(good, "rb").read()
    cases = {"magic": b"GGML" + data[4:], "version": data[:4] + (9).to_bytes(4, "little") + data[8:],
             "header": data[:40], "data": data[:len(data) - 4096]}
    for word, blob in cases.items():
        p = str(tmp_path / f"{word}.gguf")
        open(p, "wb").write(blob)
        with pytest.raises(GGufError):
            GGufFile(p)
    open(str(tmp_path / "empty.gguf"), "wb").close()
    with pytest.raises(GGufError):
        GGufFile(str(tmp_path / "empty.gguf"))
