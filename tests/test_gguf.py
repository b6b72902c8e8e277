"""GGUF container reader and writer: checked against the independent `gguf` Python package (both directions), against
hand-built files, and on malformed input.  No GPU needed: parsing is host code of the shared library."""
import os
import struct

import numpy as np
import pytest

from inferi_b200 import gguf as G
from inferi_b200 import quant
from inferi_b200._lib import InferiError
from inferi_b200.llama2 import LAYER_MATS, Llama2Config, synth_weights

gguf_py = pytest.importorskip("gguf")

TINY = Llama2Config(256, 512, 2, 4, 2, 512, 64, 500000.0, 1e-5)
RECIPE = dict(attn_q=quant.Q4_K, attn_k=quant.Q5_K, attn_v=quant.Q8_0, attn_output=quant.Q4_K, ffn_gate=quant.Q4_K, ffn_up=quant.Q4_K,
              ffn_down=quant.Q6_K, token_embd=quant.Q4_K, output=quant.Q8_0)


@pytest.fixture(scope="module")
def tiny_file(tmp_path_factory):
    w = synth_weights(TINY, seed=11, recipe=RECIPE)
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    G.write_llama_gguf(path, TINY, w, tokens=[f"<t{i}>" for i in range(TINY.vocab_size)])
    return path, w


def test_reader_matches_the_independent_reader_on_our_file(tiny_file):
    path, w = tiny_file
    ours = G.Gguf(path)
    ref = gguf_py.GGUFReader(path)
    assert ours.version == 3 and ours.alignment == 32
    assert ours.n_tensors == len(ref.tensors) == 3 + 9 * TINY.num_hidden_layers
    assert ours.tensor_names() == [t.name for t in ref.tensors]
    for t in ref.tensors:
        mine = ours.tensor(t.name)
        assert mine["type"] == int(t.tensor_type)
        assert mine["offset"] == int(t.data_offset)
        assert mine["nbytes"] == int(t.n_bytes)
        assert list(reversed(mine["shape"])) == [int(d) for d in t.shape]          # the file stores dimensions fastest first
        assert np.array_equal(mine["data"], np.asarray(t.data).reshape(-1).view(np.uint8))
    # the bytes are the checkpoint's
    assert np.array_equal(ours.tensor("blk.1.ffn_down.weight")["data"], w["layers"][1]["ffn_down"][1].numpy().reshape(-1))
    assert np.array_equal(ours.tensor("blk.0.attn_norm.weight")["data"].view(np.float32), w["layers"][0]["attn_norm"].numpy())
    # metadata
    keys = dict(ours.keys())
    assert set(keys) == {f.name for f in ref.fields.values() if not f.name.startswith("GGUF.")}
    assert ours.get("general.architecture") == "llama"
    assert ours.get("llama.block_count") == TINY.num_hidden_layers
    assert ours.get("llama.rope.freq_base") == pytest.approx(500000.0)
    toks = ours.get("tokenizer.ggml.tokens")
    assert len(toks) == TINY.vocab_size and toks[0] == "<t0>" and toks[-1] == f"<t{TINY.vocab_size - 1}>"
    cfg = ours.llama_config()
    assert cfg.rms_norm_eps == float(np.float32(TINY.rms_norm_eps)) and cfg.rope_theta == TINY.rope_theta   # f32 in the file
    cfg.rms_norm_eps = TINY.rms_norm_eps
    assert cfg == TINY
    ours.close()


def test_reader_on_a_file_written_by_the_independent_writer(tmp_path):
    path = str(tmp_path / "theirs.gguf")
    wr = gguf_py.GGUFWriter(path, "llama")
    wr.add_uint32("llama.block_count", 3)
    wr.add_float32("llama.rope.freq_base", 12345.5)
    wr.add_string("general.name", "näme")
    wr.add_bool("some.flag", True)
    wr.add_int32("some.negative", -7)
    wr.add_array("some.ints", [1, 2, 3, 4])
    wr.add_array("some.strings", ["a", "bc", ""])
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    blocks = quant.random_blocks(quant.Q4_K, 8, 512, seed=3)
    wr.add_tensor("a.weight", a)
    wr.add_tensor("q.weight", np.ascontiguousarray(blocks), raw_dtype=gguf_py.GGMLQuantizationType.Q4_K)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    g = G.Gguf(path)
    assert g.get("llama.block_count") == 3
    assert g.get("llama.rope.freq_base") == pytest.approx(12345.5)
    assert g.get("general.name") == "näme"
    assert g.get("some.flag") is True
    assert g.get("some.negative") == -7
    assert g.get("some.ints").tolist() == [1, 2, 3, 4]
    assert g.get("some.strings") == ["a", "bc", ""]
    t = g.tensor("a.weight")
    assert t["type"] == 0 and t["shape"] == (4, 6) and np.array_equal(t["data"].view(np.float32).reshape(4, 6), a)
    q = g.tensor("q.weight")
    assert q["type"] == quant.Q4_K and q["shape"] == (8, 512) and np.array_equal(q["data"], blocks.reshape(-1))
    with pytest.raises(InferiError):
        g.tensor("missing")
    with pytest.raises(InferiError):
        g.llama_config()                      # embedding_length and friends are absent
    g.close()


def test_defaults_alignment_and_in_memory_open(tmp_path):
    path = str(tmp_path / "d.gguf")
    meta = [("llama.embedding_length", G.U32, 256), ("llama.feed_forward_length", G.U32, 512), ("llama.block_count", G.U32, 1),
            ("llama.attention.head_count", G.U32, 4), ("llama.attention.head_count_kv", G.U32, 2), ("llama.context_length", G.U64, 32)]
    emb = quant.random_blocks(quant.Q8_0, 64, 256, seed=1)
    G.write_gguf(path, meta, [("token_embd.weight", quant.Q8_0, (64, 256), emb.tobytes())], alignment=64)
    data = open(path, "rb").read()
    g = G.Gguf(data=data)
    assert g.alignment == 64 and g.tensor("token_embd.weight")["offset"] % 64 == 0
    cfg = g.llama_config()
    assert cfg.vocab_size == 64                                   # no tokenizer in the file: rows of token_embd
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == pytest.approx(1e-6)   # defaults of the reference
    assert cfg.max_position_embeddings == 32                      # a u64 value is accepted where the reference wants u32
    g.close()


@pytest.mark.parametrize("damage", ["magic", "version", "truncated_meta", "truncated_table", "rank5", "past_eof", "bad_type", "huge_count"])
def test_malformed_files_are_errors(tmp_path, damage):
    path = str(tmp_path / "ok.gguf")
    blk = quant.random_blocks(quant.Q4_K, 4, 256, seed=2)
    G.write_gguf(path, [("k", G.U32, 1), ("s", G.STRING, "hello")], [("w", quant.Q4_K, (4, 256), blk.tobytes())])
    good = bytearray(open(path, "rb").read())
    G.Gguf(data=bytes(good)).close()
    bad = bytearray(good)
    if damage == "magic":
        bad[0] ^= 0xFF
    elif damage == "version":
        bad[4:8] = struct.pack("<I", 9)
    elif damage == "truncated_meta":
        bad = bad[:30]
    elif damage == "truncated_table":
        bad = bad[:good.index(b"w", 40) + 6]
    elif damage == "rank5":
        i = good.index(struct.pack("<Q", 1) + b"w") + 9
        bad[i:i + 4] = struct.pack("<I", 5)
    elif damage == "past_eof":
        bad = bad[:len(bad) - 200]
    elif damage == "bad_type":
        i = good.index(_key("k")) + len(_key("k"))
        bad[i:i + 4] = struct.pack("<I", 77)
    elif damage == "huge_count":
        bad[8:16] = struct.pack("<Q", 1 << 60)
    with pytest.raises(InferiError):
        G.Gguf(data=bytes(bad))


def _key(k: str) -> bytes:
    return struct.pack("<Q", len(k)) + k.encode()
