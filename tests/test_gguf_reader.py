"""GGUF container reader against files written by the third-party ``gguf`` package (its writer and its own
reader are the witnesses; the reference has no GGUF code).  CPU only."""
import os
import struct

import numpy as np
import pytest
import torch

import oracle
from tattletale_b200 import FMT_Q4_K, FMT_Q6_K, FMT_Q8_0
from tattletale_b200.gguf_reader import GGUFError, GGUFFile

gguf = pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def sample(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("gguf") / "sample.gguf")
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, (48, 512)).astype(np.float32)
    tensors = {
        "blk.0.attn_q.weight": (oracle.quantize(oracle.Q8_0, w), gguf.GGMLQuantizationType.Q8_0),
        "blk.0.ffn_up.weight": (oracle.quantize(oracle.Q4_K, w), gguf.GGMLQuantizationType.Q4_K),
        "output.weight": (oracle.quantize(oracle.Q6_K, w), gguf.GGMLQuantizationType.Q6_K),
    }
    norm = rng.normal(1, 0.02, 512).astype(np.float32)
    wr = gguf.GGUFWriter(path, "llama")
    wr.add_uint32("llama.block_count", 1)
    wr.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    wr.add_string("general.name", "sample")
    wr.add_array("tokenizer.ggml.scores", [0.5, -1.0, 2.0])
    wr.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    for name, (blocks, qt) in tensors.items():
        wr.add_tensor(name, blocks, raw_dtype=qt)
    wr.add_tensor("blk.0.attn_norm.weight", norm)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return path, tensors, norm, w


def test_tensor_table_and_bytes_match_the_witness(sample):
    path, tensors, norm, _ = sample
    theirs = {t.name: t for t in gguf.GGUFReader(path).tensors}
    with GGUFFile(path) as f:
        assert set(f.tensors) == set(theirs)
        for name, (blocks, qt) in tensors.items():
            info = f.tensors[name]
            assert info.shape == (48, 512) and info.ggml_type == int(qt)
            assert info.nbytes == blocks.size == int(theirs[name].n_bytes)
            got = f.blocks(name)
            assert got.dtype == torch.uint8 and tuple(got.shape) == blocks.shape
            assert np.array_equal(got.numpy(), blocks)
            assert np.array_equal(f.raw(name), np.asarray(theirs[name].data).reshape(-1).view(np.uint8))
        assert np.array_equal(f.array("blk.0.attn_norm.weight"), norm)
        del got


def test_metadata(sample):
    path = sample[0]
    with GGUFFile(path) as f:
        assert f.version == 3 and f.alignment == 32
        assert f.metadata["general.architecture"] == "llama"
        assert f.metadata["llama.block_count"] == 1
        assert abs(f.metadata["llama.attention.layer_norm_rms_epsilon"] - 1e-5) < 1e-12
        assert f.metadata["general.name"] == "sample"
        assert np.allclose(f.metadata["tokenizer.ggml.scores"], [0.5, -1.0, 2.0])
        assert f.metadata["tokenizer.ggml.tokens"] == ["a", "bc", "def"]


def test_blocks_decode_to_the_weights(sample):
    """The views are canonical blocks: the checker dequantizes them back to the encoder's values."""
    path, tensors, _, w = sample
    with GGUFFile(path) as f:
        for name, ofmt, tol in (("blk.0.attn_q.weight", oracle.Q8_0, 0.01), ("blk.0.ffn_up.weight", oracle.Q4_K, 0.12),
                                ("output.weight", oracle.Q6_K, 0.03)):
            deq = oracle.dequantize(ofmt, f.blocks(name).numpy().copy())
            assert np.linalg.norm(deq - w) / np.linalg.norm(w) < tol


def test_errors(sample, tmp_path):
    path = sample[0]
    with GGUFFile(path) as f:
        with pytest.raises(GGUFError):
            f.blocks("nope")
        with pytest.raises(GGUFError):
            f.blocks("blk.0.attn_norm.weight")  # F32, not a block format
        with pytest.raises(GGUFError):
            f.array("output.weight")            # quantized: use blocks()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 40)
    with pytest.raises(GGUFError):
        GGUFFile(str(bad))
    data = bytearray(open(path, "rb").read())
    struct.pack_into("<I", data, 4, 9)          # unknown version
    bad.write_bytes(bytes(data))
    with pytest.raises(GGUFError):
        GGUFFile(str(bad))
    bad.write_bytes(open(path, "rb").read()[:-64])  # truncated data section
    with pytest.raises(GGUFError):
        GGUFFile(str(bad))


def test_format_map():
    from tattletale_b200.gguf_reader import TTQ_FORMATS

    assert TTQ_FORMATS == {8: FMT_Q8_0, 12: FMT_Q4_K, 14: FMT_Q6_K}
