"""The GGUF v3 reader behind the C ABI (rq_gguf_*), on files written the way the reference's own test writes one
(.github/runtime/suite.rs:127-214). No GPU: the reader only maps and parses."""
import ctypes as C
import struct

import numpy as np
import pytest

from tests import gguf_writer as gw
from tests import oracle_lib as ol


def stepper_checkpoint(path):
    """The reference's stepper checkpoint: F32 scalars and small matrices plus one Q8_0 table of four rows
    (d = 0x2400, codes 32, 96, -80, 48), the metadata pairs in the reference's order."""
    tensors = [("token_embd.weight", [1, 2], 0, np.array([1.0, 2.0], np.float32)), ("blk.0.ffn_gate.weight", [1, 1], 0, np.array([2.0], np.float32)),
               ("output.weight", [1, 2], 0, np.array([1.0, -1.0], np.float32))]
    table = b"".join(struct.pack("<H", 0x2400) + bytes([code & 0xFF] * 32) for code in (32, 96, -80, 48))
    tensors.append(("ngram.table", [32, 4], 8, np.frombuffer(table, np.uint8)))
    tensors.append(("blk.0.ple_key.weight", [64, 1], 0, np.full(64, 0.01, np.float32)))
    metadata = [("general.architecture", gw.KIND_STRING, "llama"), ("tokenizer.ggml.model", gw.KIND_STRING, "gpt2"),
                ("llama.context_length", gw.KIND_U32, 160), ("tokenizer.ggml.eos_token_id", gw.KIND_U32, 1), ("tokenizer.ggml.add_bos_token", gw.KIND_BOOL, False),
                ("tokenizer.ggml.tokens", gw.KIND_ARRAY, (gw.KIND_STRING, ["a", "b"])), ("tokenizer.ggml.merges", gw.KIND_ARRAY, (gw.KIND_STRING, [])),
                ("llama.rope.freq_base", gw.KIND_F32, 10000.0), ("some.i64", gw.KIND_I64, -5), ("some.f64", gw.KIND_F64, 0.25),
                ("nested", gw.KIND_ARRAY, (gw.KIND_ARRAY, [(gw.KIND_U8, [1, 2]), (gw.KIND_U8, [])]))]
    gw.write_gguf(path, metadata, tensors)
    return tensors


def test_stepper_checkpoint_round_trip(tmp_path, oracle):
    import recipe_dev_b200 as rq

    path = tmp_path / "stepper.gguf"
    written = stepper_checkpoint(path)
    g = rq.Gguf(path)
    got = g.tensors()
    assert [t["name"] for t in got] == [t[0] for t in written]
    assert [t["shape"] for t in got] == [t[1] for t in written]
    assert [t["type"] for t in got] == [t[2] for t in written]
    for t, w in zip(got, written):
        payload = np.ascontiguousarray(w[3]).view(np.uint8).reshape(-1)
        assert t["bytes"] == payload.size
        assert np.array_equal(g.data(t["name"]), payload)
    # the Q8_0 table decodes to the reference's constants (suite.rs:191-194)
    rows = oracle.dequantize(ol.Q8_0, g.data("ngram.table")).reshape(4, 32)
    assert np.array_equal(rows, np.repeat(np.array([[0.5], [1.5], [-1.25], [0.75]], np.float32), 32, axis=1))
    # metadata: file order, every width as the file chose it
    assert g.keys()[:3] == ["general.architecture", "tokenizer.ggml.model", "llama.context_length"]
    assert g.text("general.architecture") == "llama" and g.integer("llama.context_length") == 160 and g.integer("tokenizer.ggml.add_bos_token") == 0
    assert g.array_text("tokenizer.ggml.tokens") == ["a", "b"] and g.array_text("tokenizer.ggml.merges") == []
    assert g.float("llama.rope.freq_base") == 10000.0 and g.float("some.f64") == 0.25
    assert g.lib.rq_gguf_meta_kind(g.handle, b"nested") == 9 and g.lib.rq_gguf_meta_array_length(g.handle, b"nested") == 2
    with pytest.raises(rq.RqError):
        g.integer("some.i64")  # negative: not a count
    with pytest.raises(rq.RqError):
        g.integer("absent.key")
    assert g.lib.rq_gguf_find(g.handle, b"nope") == -1
    g.close()


def test_alignment_and_block_checks(tmp_path, oracle):
    import recipe_dev_b200 as rq

    blocks = oracle.quantize(ol.Q4_K, oracle.normal(81, 0, 8 * 512, 0.02))
    # a declared alignment of 64 moves the data section
    path = tmp_path / "a64.gguf"
    gw.write_gguf(path, [("k", gw.KIND_U32, 1)], [("w", [512, 8], 12, blocks), ("v", [4], 0, np.arange(4, dtype=np.float32))], alignment=64, declare_alignment=True)
    g = rq.Gguf(path)
    assert np.array_equal(g.data("w"), blocks) and np.array_equal(g.data("v").view(np.float32), np.arange(4, dtype=np.float32))
    g.close()
    lib = rq.load_library()
    out = C.c_void_p()

    def refuses(p, text):
        rc = lib.rq_gguf_open(str(p).encode(), C.byref(out))
        assert rc == -1 and text in lib.rq_last_error().decode(), lib.rq_last_error()

    # not GGUF, wrong version, truncated header, element count that cuts a block, tensor past the end, bad alignment
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + bytes(60))
    refuses(bad, "is not a GGUF file")
    gw.write_gguf(bad, [], [], version=2)
    refuses(bad, "version 2")
    whole = path.read_bytes()
    bad.write_bytes(whole[:40])
    refuses(bad, "truncated")
    gw.write_gguf(bad, [], [("w", [100, 3], 12, blocks[:144 * 2])])
    refuses(bad, "not a multiple of its 256-element block")
    gw.write_gguf(bad, [], [("w", [512, 16], 12, blocks)])
    refuses(bad, "runs past the end")
    gw.write_gguf(bad, [("general.alignment", gw.KIND_U32, 48)], [])
    refuses(bad, "alignment 48")
    gw.write_gguf(bad, [], [("w", [32], 99, np.zeros(32, np.uint8))])
    refuses(bad, "type 99")
    refuses(tmp_path / "missing.gguf", "cannot open")


def test_split_model(tmp_path, oracle):
    import recipe_dev_b200 as rq

    a = oracle.quantize(ol.Q8_0, oracle.normal(82, 0, 4 * 64, 0.02))
    b = oracle.quantize(ol.Q6_K, oracle.normal(82, 1, 2 * 256, 0.02))
    first, second = tmp_path / "m-00001-of-00002.gguf", tmp_path / "m-00002-of-00002.gguf"
    gw.write_gguf(first, [("split.count", gw.KIND_U16, 2), ("split.no", gw.KIND_U16, 0), ("split.tensors.count", gw.KIND_I32, 2)], [("a", [64, 4], 8, a)])
    gw.write_gguf(second, [("split.count", gw.KIND_U16, 2), ("split.no", gw.KIND_U16, 1)], [("b", [256, 2], 14, b)])
    g = rq.Gguf(first)
    assert [t["name"] for t in g.tensors()] == ["a", "b"]
    assert np.array_equal(g.data("a"), a) and np.array_equal(g.data("b"), b)
    g.close()
    # a shard that is not the one its name says
    gw.write_gguf(second, [("split.count", gw.KIND_U16, 2), ("split.no", gw.KIND_U16, 0)], [("b", [256, 2], 14, b)])
    with pytest.raises(rq.RqError, match="expected shard 1"):
        rq.Gguf(first)
