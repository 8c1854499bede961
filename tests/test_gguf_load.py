"""GGUF ingestion: the reader against files written by the `gguf` package, the nibble repack against
the checker's two dequantizers, and (GPU) a loaded shard through the kernels."""
import os

import numpy as np
import pytest

from bpd_substrate_b200 import gguf_load, synth

gguf = pytest.importorskip("gguf")


def u32(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def model_file(tmp_path_factory):
    """A small GGUF file with Q4_K, Q8_0 and F32 tensors and metadata of every kind the reader parses."""
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    rng = np.random.default_rng(123)
    tensors = {
        "blk.0.ffn_gate.weight": (synth.q4k_matrix(64, 512, rng).reshape(64, 512 // 256 * 144), gguf.GGMLQuantizationType.Q4_K),
        "blk.0.attn_q.weight": (synth.q8_0_matrix(48, 256, rng).reshape(48, 256 // 32 * 34), gguf.GGMLQuantizationType.Q8_0),
        "blk.0.attn_norm.weight": (rng.standard_normal(256, dtype=np.float32), None),
        "output.weight": (synth.q4k_matrix(32, 256, rng).reshape(32, 144), gguf.GGMLQuantizationType.Q4_K),
    }
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", 1)
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_bool("general.some_flag", True)
    w.add_string("general.name", "tiny test model")
    w.add_array("tokenizer.ggml.tokens", ["<s>", "</s>", "hello", "wörld"])
    w.add_array("tokenizer.ggml.token_type", [1, 1, 0, 0])
    w.add_uint64("general.big", 1 << 40)
    for name, (arr, qt) in tensors.items():
        w.add_tensor(name, arr, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, tensors


def test_reader_recovers_metadata_and_tensor_bytes(model_file):
    path, tensors = model_file
    g = gguf_load.GgufFile(path)
    try:
        assert g.version >= 2
        assert g.metadata["llama.block_count"] == 1
        assert abs(g.metadata["llama.attention.layer_norm_rms_epsilon"] - 1e-5) < 1e-12
        assert g.metadata["general.some_flag"] is True
        assert g.metadata["general.name"] == "tiny test model"
        assert g.metadata["tokenizer.ggml.tokens"] == ["<s>", "</s>", "hello", "wörld"]
        assert g.metadata["tokenizer.ggml.token_type"] == [1, 1, 0, 0]
        assert g.metadata["general.big"] == 1 << 40
        assert set(g.tensors) == set(tensors)
        t = g.tensors["blk.0.ffn_gate.weight"]
        assert (t.type, t.dims, t.rows, t.row_bytes) == (gguf_load.TYPE_Q4_K, (512, 64), 64, 288)
        t = g.tensors["blk.0.attn_q.weight"]
        assert (t.type, t.dims, t.rows, t.row_bytes) == (gguf_load.TYPE_Q8_0, (256, 48), 48, 272)
        for name, (arr, _) in tensors.items():
            assert np.array_equal(g.raw(name), np.ascontiguousarray(arr).view(np.uint8).ravel()), name
        # a row shard is a contiguous byte range
        whole = g.raw("blk.0.ffn_gate.weight")
        assert np.array_equal(g.raw("blk.0.ffn_gate.weight", 16, 32), whole[16 * 288:32 * 288])
        with pytest.raises(ValueError):
            g.raw("blk.0.ffn_gate.weight", 0, 65)
        # the package's own reader sees the same table
        theirs = {t.name: (tuple(int(d) for d in t.shape), int(t.tensor_type), int(t.n_bytes)) for t in gguf.GGUFReader(path).tensors}
        mine = {n: (t.dims, t.type, t.nbytes) for n, t in g.tensors.items()}
        assert mine == theirs
    finally:
        g.close()


def test_reader_rejects_other_files(tmp_path):
    p = tmp_path / "not.gguf"
    p.write_bytes(b"GGML" + bytes(64))
    with pytest.raises(ValueError):
        gguf_load.GgufFile(str(p))


def test_nibble_repack_is_exact_and_invertible(oracle):
    raw = synth.q4k_blocks(333, 9)                       # read as if it were in ggml's order
    bpd = gguf_load.repack_q4k_ggml_to_bpd(raw)
    assert np.array_equal(gguf_load.repack_q4k_bpd_to_ggml(bpd), raw)
    blocks, moved = raw.reshape(-1, 144), bpd.reshape(-1, 144)
    assert np.array_equal(blocks[:, :16], moved[:, :16])     # d, dmin, scales and mins stay
    assert not np.array_equal(blocks[:, 16:], moved[:, 16:])
    # same numbers out of the two dequantizers, and out of the gguf package's own
    want = oracle.dequant_q4k(raw, 1)
    assert np.array_equal(u32(oracle.dequant_q4k(bpd, 0)), u32(want))
    theirs = gguf.quants.dequantize(raw.reshape(-1, 144), gguf.GGMLQuantizationType.Q4_K).ravel()
    assert np.array_equal(u32(theirs), u32(want))


@pytest.mark.gpu
def test_loaded_shards_run_through_the_kernels(lib, oracle, model_file):
    from tests.util import Dev, normwise
    path, tensors = model_file
    g = gguf_load.GgufFile(path)
    try:
        x = np.random.default_rng(5).standard_normal(512, dtype=np.float32)
        dX = Dev(lib, x)
        raw = g.raw("blk.0.ffn_gate.weight")
        xq = oracle.quant_q8_K(x)
        for rank in (0, 1):
            want = oracle.qmatmul_q4k_q8k(raw[rank * 32 * 288:(rank + 1) * 32 * 288], xq, 32, 512, 1)[1]
            for repack in (False, True):
                ptr, rows, cols, ttype, layout = g.to_device(lib, "blk.0.ffn_gate.weight", rank, 2, repack)
                assert (rows, cols, ttype, layout) == (32, 512, gguf_load.TYPE_Q4_K, 0 if repack else 1)
                dO = Dev(lib, nbytes=rows * 4)
                assert lib.bpd_qmm_q4k_q8k_cuda(ptr, dX.ptr, dO.ptr, 1, rows, cols, layout, 0, None, None) == 0
                lib.bpdq_sync()
                assert normwise(dO.read(np.float32), want) <= 1e-5
                lib.bpdq_free(ptr)
        # Q8_0 shard through the Q8_0 product
        x8 = x[:256].copy()
        ptr, rows, cols, ttype, layout = g.to_device(lib, "blk.0.attn_q.weight")
        dX8, dO = Dev(lib, x8), Dev(lib, nbytes=rows * 4)
        assert lib.bpd_qmatmul_q8_0_cuda(ptr, dX8.ptr, dO.ptr, 1, rows, cols, None) == 0
        lib.bpdq_sync()
        assert normwise(dO.read(np.float32), oracle.qmatmul_q8_0(g.raw("blk.0.attn_q.weight"), x8, 1, rows, cols)) <= 1e-5
        lib.bpdq_free(ptr)
        assert lib.bpdq_last_status() == 0
    finally:
        g.close()
