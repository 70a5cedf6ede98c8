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


# ---- shards ------------------------------------------------------------------------------------------------------
def write_raw_gguf(path, metadata, tensors):
    """A GGUF file written by hand (version 3): metadata {key: ("u32" | "u16" | "f32" | "str", value)}, tensors
    {name: torch tensor of float32 or bfloat16}.  The ``gguf`` package always adds general.architecture, which the
    later shards of a model must not repeat."""
    import struct

    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    kinds = {"u16": (2, "<H"), "u32": (4, "<I"), "f32": (6, "<f")}
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for k, (kind, v) in metadata.items():
        head += s(k) + (struct.pack("<I", 8) + s(v) if kind == "str" else
                        struct.pack("<I", kinds[kind][0]) + struct.pack(kinds[kind][1], v))
    blobs, off = [], 0
    for name, t in tensors.items():
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).contiguous().numpy().tobytes()
        head += s(name) + struct.pack("<I", t.dim()) + b"".join(struct.pack("<Q", d) for d in reversed(t.shape))
        head += struct.pack("<IQ", 30 if t.dtype == torch.bfloat16 else 0, off)
        blobs.append(raw + b"\0" * (-len(raw) % 32))
        off += len(blobs[-1])
    with open(path, "wb") as f:
        f.write(head + b"\0" * (-len(head) % 32) + b"".join(blobs))
    return path


def _sharded(tmp_path, cfg, tensors, stem="model", count=3, extra_meta=None, repeat=None):
    """The model cut into ``count`` shards: all metadata in the first, split.* keys in every one."""
    m = LlamaMeta.from_dict(cfg)
    meta = {"general.architecture": ("str", "llama"), "llama.block_count": ("u32", m.nblk),
            "llama.embedding_length": ("u32", m.d), "llama.attention.head_count": ("u32", m.nh),
            "llama.attention.head_count_kv": ("u32", m.nkvh), "llama.rope.dimension_count": ("u32", m.dh),
            "llama.feed_forward_length": ("u32", m.di), "llama.expert_count": ("u32", m.nexp),
            "llama.expert_used_count": ("u32", m.nexp_use), "llama.context_length": ("u32", m.nctx),
            "llama.vocab_size": ("u32", m.nvoc), "llama.attention.layer_norm_rms_epsilon": ("f32", m.epsilon),
            "llama.rope.freq_base": ("f32", m.theta), "rope_pairing": ("str", m.rope_pairing)}
    names = list(tensors)
    paths = []
    for i in range(count):
        part = {n: tensors[n] for n in names[i::count]}
        if repeat and i == count - 1:
            part[repeat] = tensors[repeat]
        md = dict(meta) if i == 0 else {}
        md.update({"split.no": ("u16", i), "split.count": ("u16", count), "general.alignment": ("u32", 32)})
        if extra_meta and i == count - 1:
            md.update(extra_meta)
        paths.append(write_raw_gguf(str(tmp_path / f"{stem}-{i + 1:05d}-of-{count:05d}.gguf"), md, part))
    return paths


def test_a_sharded_model_loads_from_any_of_its_shards(tmp_path):
    rules = tensor_plan(LlamaMeta.from_dict(TINY_A))
    tensors = random_file_tensors(rules, 4, torch.bfloat16, std=0.1)
    whole = load_weights(write_raw_gguf(str(tmp_path / "whole.gguf"), {}, tensors), rules, torch.float32, CPU)
    paths = _sharded(tmp_path, TINY_A, tensors)
    for p in (paths[0], paths[2]):
        meta = LlamaMeta.from_dict(tb.read_config(p))
        assert (meta.nblk, meta.nexp, meta.nvoc) == (2, 4, 256)
        got = load_weights(p, tensor_plan(meta), torch.float32, CPU)
        assert sorted(got) == sorted(whole) and all(torch.equal(got[k], whole[k]) for k in whole)


def test_shard_faults_are_named(tmp_path):
    from transformer_b200.weights.gguf import open_gguf, shard_paths
    rules = tensor_plan(LlamaMeta.from_dict(TINY_A))
    tensors = random_file_tensors(rules, 4, torch.bfloat16, std=0.1)
    assert shard_paths("/x/m.gguf") == ["/x/m.gguf"] and shard_paths("/x/m-00001-of-00001.gguf") == ["/x/m-00001-of-00001.gguf"]
    assert [p[-19:] for p in shard_paths("/x/m-00002-of-00003.gguf")] == [f"{i:05d}-of-00003.gguf" for i in (1, 2, 3)]
    with pytest.raises(GGufError, match="outside 1..3"):
        shard_paths("/x/m-00004-of-00003.gguf")
    paths = _sharded(tmp_path, TINY_A, tensors, stem="gone")
    import os
    os.remove(paths[1])
    with pytest.raises(GGufError, match="shards missing: gone-00002-of-00003.gguf"):
        open_gguf(paths[0])
    paths = _sharded(tmp_path, TINY_A, tensors, stem="twice", repeat="token_embd.weight")
    with pytest.raises(GGufError, match="shard 3 .*tensor 'token_embd.weight' is in an earlier shard"):   # gguf/src/lib.rs:112-124
        open_gguf(paths[1])
    paths = _sharded(tmp_path, TINY_A, tensors, stem="key", extra_meta={"llama.block_count": ("u32", 2)})
    with pytest.raises(GGufError, match="shard 3 .*metadata key 'llama.block_count' is in an earlier shard"):   # :99-110
        open_gguf(paths[0])
