"""GGUF container: write -> read round trips, the rules of the reference's reader
(fusor-ml/gguf/src/lib.rs:559-613) and its error cases. Host code only."""
import struct

import numpy as np
import pytest

from kalosm_b200 import gguf
from oracle import oracle as O


def test_round_trip_metadata_tensors_and_alignment(tmp_path):
    q = O.random_qweights(1, 0.02, 4 * 512, O.Q4K)
    v = np.arange(6, dtype=np.float32)
    md = {"general.architecture": (gguf.STRING, "llama"), "a.u8": (gguf.U8, 200), "a.i8": (gguf.I8, -3),
          "a.u16": (gguf.U16, 65535), "a.i16": (gguf.I16, -2), "a.u32": (gguf.U32, 7), "a.i32": (gguf.I32, -7),
          "a.f32": (gguf.F32, 1.5), "a.bool": (gguf.BOOL, True), "a.u64": (gguf.U64, 1 << 40), "a.i64": (gguf.I64, -(1 << 40)),
          "a.f64": (gguf.F64, 2.25), "a.str": (gguf.STRING, "héllo\0\0"),
          "a.arr": (gguf.ARRAY, (gguf.STRING, ["x", "yz"])), "a.nested": (gguf.ARRAY, (gguf.ARRAY, [(gguf.U32, [1, 2]), (gguf.U32, [])]))}
    for align in (None, 64):
        path = tmp_path / f"t{align}.gguf"
        gguf.write_gguf(path, md, [("w", (4, 512), O.Q4K, q), ("v", (6,), 0, v)], alignment=align)
        g = gguf.GgufFile(path)
        assert g.version == 3 and g.alignment == (align or 32) and g.tensor_data_offset % g.alignment == 0
        assert g.metadata["a.u8"] == 200 and g.metadata["a.i8"] == -3 and g.metadata["a.i64"] == -(1 << 40)
        assert g.metadata["a.str"] == "héllo"  # trailing NULs are dropped (lib.rs:328-331)
        assert g.metadata["a.arr"] == ["x", "yz"] and g.metadata["a.nested"] == [[1, 2], []]
        assert g.metadata["a.bool"] is True and g.metadata["a.f64"] == 2.25
        assert g.tensors["w"][:2] == ((4, 512), O.Q4K)  # stored innermost first, outermost first once read
        assert np.array_equal(g.tensor_bytes("w"), q)
        assert np.array_equal(np.frombuffer(bytes(g.tensor_bytes("v")), np.float32), v)
        assert g.tensors["v"][2] % g.alignment == 0


def test_version_1_uses_32_bit_lengths(tmp_path):
    key = b"general.alignment"
    raw = gguf.MAGIC + struct.pack("<III", 1, 0, 1) + struct.pack("<I", len(key)) + key + struct.pack("<II", gguf.U32, 16)
    p = tmp_path / "v1.gguf"
    p.write_bytes(raw)
    g = gguf.GgufFile(p)
    assert g.version == 1 and g.alignment == 16 and g.tensor_data_offset % 16 == 0 and not g.tensors


@pytest.mark.parametrize("raw,what", [
    (b"GGML" + bytes(20), "magic"),
    (gguf.MAGIC + struct.pack("<IQQ", 9, 0, 0), "version"),
    (gguf.MAGIC + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 99), "value type"),
    (gguf.MAGIC + struct.pack("<IQQ", 3, 1, 0), "end of file"),
    (gguf.MAGIC + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IB", gguf.BOOL, 2), "bool"),
])
def test_malformed_files_are_errors(tmp_path, raw, what):
    p = tmp_path / "bad.gguf"
    p.write_bytes(raw)
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile(p)
    assert what in str(e.value)


def test_tensor_checks_and_llama_config(tmp_path):
    p = tmp_path / "m.gguf"
    md = {"general.architecture": (gguf.STRING, "llama"), "llama.block_count": (gguf.U32, 2),
          "llama.embedding_length": (gguf.U32, 256), "llama.feed_forward_length": (gguf.U32, 512),
          "llama.attention.head_count": (gguf.U32, 4), "llama.attention.head_count_kv": (gguf.U32, 2),
          "llama.context_length": (gguf.U32, 64), "llama.attention.layer_norm_rms_epsilon": (gguf.F32, 1e-5),
          "llama.rope.freq_base": (gguf.F32, 500000.0)}
    emb = O.random_qweights(2, 0.02, 1024 * 256, O.Q4K)
    gguf.write_gguf(p, md, [("token_embd.weight", (1024, 256), O.Q4K, emb), ("odd", (3, 100), O.Q4K, np.zeros(8, np.uint8)),
                            ("unknown", (2, 32), 31, np.zeros(8, np.uint8))])
    g = gguf.GgufFile(p)
    c = gguf.llama_config(g)
    assert c == dict(n_layer=2, hidden=256, ffn=512, n_head=4, n_kv_head=2, head_dim=64, vocab=1024, ctx=64,
                     rms_eps=pytest.approx(1e-5), rope_theta=500000.0)
    with pytest.raises(gguf.GgufError):
        g.tensor_bytes("odd")       # 100 is not a multiple of the 256-element block
    with pytest.raises(gguf.GgufError):
        g.tensor_bytes("unknown")   # ggml type outside the supported set
    with pytest.raises(KeyError):
        g.tensor_bytes("missing")
    del md["llama.block_count"]
    gguf.write_gguf(p, md, [("token_embd.weight", (1024, 256), O.Q4K, emb)])
    with pytest.raises(gguf.GgufError):
        gguf.llama_config(gguf.GgufFile(p))


def _tiny_md(**over):
    md = {"general.architecture": (gguf.STRING, "llama"), "llama.block_count": (gguf.U32, 1),
          "llama.embedding_length": (gguf.U32, 256), "llama.feed_forward_length": (gguf.U32, 512),
          "llama.attention.head_count": (gguf.U32, 4), "llama.attention.head_count_kv": (gguf.U32, 2),
          "llama.context_length": (gguf.U32, 64), "llama.attention.layer_norm_rms_epsilon": (gguf.F32, 1e-5)}
    md.update(over)
    return {k: v for k, v in md.items() if v is not None}


def test_loader_defaults_and_refusals(tmp_path):
    # what Model::from_var_source does with the same files (models/kalosm-llama/src/raw/mod.rs:377-434):
    # rope.freq_base defaults to DEFAULT_ROPE_FREQUENCY (:104, :385-388); head_count_kv is mandatory
    # (:379); other architectures need code paths this build does not have
    emb = O.random_qweights(2, 0.02, 1024 * 256, O.Q4K)
    p = tmp_path / "m.gguf"
    gguf.write_gguf(p, _tiny_md(), [("token_embd.weight", (1024, 256), O.Q4K, emb)])
    assert gguf.llama_config(gguf.GgufFile(p))["rope_theta"] == 1_000_000.0
    gguf.write_gguf(p, _tiny_md(**{"llama.attention.head_count_kv": None}), [("token_embd.weight", (1024, 256), O.Q4K, emb)])
    with pytest.raises(gguf.GgufError) as e:
        gguf.llama_config(gguf.GgufFile(p))
    assert "head_count_kv" in str(e.value)
    for arch in ("qwen2", "gemma3", "phi3"):
        md = {k.replace("llama.", arch + "."): v for k, v in _tiny_md().items()}
        md["general.architecture"] = (gguf.STRING, arch)
        gguf.write_gguf(p, md, [("token_embd.weight", (1024, 256), O.Q4K, emb)])
        with pytest.raises(gguf.GgufError) as e:
            gguf.llama_config(gguf.GgufFile(p))
        assert arch in str(e.value)
    # a file that asks for RoPE scaling is refused unless the caller supplies the scaling (no device needed:
    # the refusal comes before anything is built)
    gguf.write_gguf(p, _tiny_md(**{"llama.rope.scaling.factor": (gguf.F32, 8.0)}),
                    [("token_embd.weight", (1024, 256), O.Q4K, emb)])
    with pytest.raises(gguf.GgufError) as e:
        gguf.load_llama(None, p)
    assert "rope.scaling" in str(e.value)


def test_reader_against_the_gguf_package_writer(tmp_path):
    # the container format pinned independently of this repository's own writer: a file written by
    # the third-party `gguf` package (llama.cpp's Python writer) must read back identically
    pkg = pytest.importorskip("gguf")
    if not hasattr(pkg, "GGUFWriter"):
        pytest.skip("the installed gguf package has no writer")
    path = tmp_path / "pkg.gguf"
    w = pkg.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 3)
    w.add_float32("llama.rope.freq_base", 500000.0)
    w.add_string("general.name", "pinned")
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_bool("llama.flag", True)
    f32 = np.arange(24, dtype=np.float32).reshape(4, 6)
    q8 = O.random_qweights(3, 0.02, 8 * 64, O.Q8_0)
    q4k = O.random_qweights(4, 0.02, 2 * 512, O.Q4K)
    w.add_tensor("dense", f32)
    w.add_tensor("q8", q8.reshape(8, 64 // 32 * 34), raw_dtype=pkg.GGMLQuantizationType.Q8_0)
    w.add_tensor("q4k", q4k.reshape(2, 512 // 256 * 144), raw_dtype=pkg.GGMLQuantizationType.Q4_K)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    g = gguf.GgufFile(path)
    assert g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 3
    assert g.metadata["llama.rope.freq_base"] == 500000.0 and g.metadata["general.name"] == "pinned"
    assert g.metadata["tokenizer.ggml.tokens"] == ["a", "bc", "def"] and g.metadata["llama.flag"] is True
    assert g.tensors["dense"][:2] == ((4, 6), 0)
    assert np.array_equal(np.frombuffer(bytes(g.tensor_bytes("dense")), np.float32).reshape(4, 6), f32)
    assert g.tensors["q8"][:2] == ((8, 64), O.Q8_0) and np.array_equal(g.tensor_bytes("q8"), q8)
    assert g.tensors["q4k"][:2] == ((2, 512), O.Q4K) and np.array_equal(g.tensor_bytes("q4k"), q4k)


def test_five_bit_tensors_round_trip_and_shard(tmp_path):
    # Q5_0 (22-byte blocks) and Q5_K (176-byte blocks) through the container and the tensor-parallel
    # cuts: row shards and column shards dequantise (oracle) to the matching part of the whole matrix
    import fixtures as F
    from kalosm_b200 import tp
    n, k = 8, 1024
    mats = {O.Q5_0: F.random_q5_weights(3, 0.02, n, k, O.Q5_0), O.Q5K: F.random_q5_weights(4, 0.02, n, k, O.Q5K)}
    path = tmp_path / "q5.gguf"
    gguf.write_gguf(path, {"general.architecture": (gguf.STRING, "llama")},
                    [("a", (n, k), O.Q5_0, mats[O.Q5_0]), ("b", (n, k), O.Q5K, mats[O.Q5K])])
    g = gguf.GgufFile(path)
    for name, ty in (("a", O.Q5_0), ("b", O.Q5K)):
        assert g.tensors[name][:2] == ((n, k), ty)
        assert g.tensor_nbytes(name) == O.nbytes_for(ty, n * k)
        raw = np.frombuffer(bytes(g.tensor_bytes(name)), np.uint8)
        assert np.array_equal(raw, mats[ty])
        whole = O.dequantize(raw, ty, n * k).reshape(n, k)
        for rank in range(2):
            part, shape = tp.shard("attn_q", raw, ty, (n, k), rank, 2)
            assert shape == (n // 2, k)
            assert np.array_equal(O.dequantize(part, ty, part.size // O.BLOCK[ty][1] * O.BLOCK[ty][0]).reshape(shape),
                                  whole[rank * n // 2:(rank + 1) * n // 2])
            part, shape = tp.shard("ffn_down", raw, ty, (n, k), rank, 2)
            assert shape == (n, k // 2)
            assert np.array_equal(O.dequantize(part, ty, part.size // O.BLOCK[ty][1] * O.BLOCK[ty][0]).reshape(shape),
                                  whole[:, rank * k // 2:(rank + 1) * k // 2])
