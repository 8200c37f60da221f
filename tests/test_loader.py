"""GGUF file -> QuantizedArrays: write a tiny file with gguf-py's GGUFWriter, read it back with
load_gguf.  Follows the reference's round-trip test (tests/test_loader.py:20-85 there): F32, F16,
Q4_K, Q6_K, Q8_0 and a 3-D IQ4_XS tensor; metadata, names/shapes/qtypes, the tensor filter and
the default dtype.  Everything about the container is checked on the CPU; decoding the loaded
payloads bit-exactly needs the device and is marked gpu.
"""
import zlib

import gguf
import numpy as np
import pytest
import torch
from gguf import GGUFWriter
from gguf.constants import GGML_QUANT_SIZES
from gguf.constants import GGMLQuantizationType as QT

import gguf_jax_b200 as gj
from gguf_jax_b200 import synth
from oracle import oracle as O

BLOCK_TENSORS = {
    "blk.0.attn_q.weight": (QT.Q4_K, (512, 256)),
    "blk.0.attn_k.weight": (QT.Q6_K, (256, 256)),
    "blk.0.ffn_up.weight": (QT.Q8_0, (128, 64)),
    "blk.0.ffn_down.weight": (QT.IQ4_XS, (2, 4, 256)),
}


def _payload(name, qtype, shape):
    bs, ts = GGML_QUANT_SIZES[qtype]
    rows = int(np.prod(shape[:-1]))
    blocks = synth.random_blocks(qtype, rows * (shape[-1] // bs), seed=zlib.crc32(name.encode()))
    return blocks.reshape(*shape[:-1], shape[-1] // bs * ts)


@pytest.fixture(scope="module")
def tiny_gguf(tmp_path_factory):
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    wr = GGUFWriter(str(path), arch="llama")
    wr.add_name("tiny test model")
    wr.add_uint32("test.some_number", 42)
    wr.add_float32("test.some_float", 0.5)
    wr.add_array("test.some_list", [1, 2, 3])
    rng = np.random.default_rng(0)
    want = {}
    f32 = rng.normal(size=(8, 16)).astype(np.float32)
    wr.add_tensor("output_norm.weight", f32)
    want["output_norm.weight"] = (QT.F32, f32, f32.view(np.uint8))
    f16 = rng.normal(size=(8, 16)).astype(np.float16)
    wr.add_tensor("blk.0.attn_norm.weight", f16)
    want["blk.0.attn_norm.weight"] = (QT.F16, f16.astype(np.float32), f16.view(np.uint8))
    for name, (qtype, shape) in BLOCK_TENSORS.items():
        raw = _payload(name, qtype, shape)
        wr.add_tensor(name, raw, raw_dtype=qtype)
        want[name] = (qtype, gguf.quants.dequantize(raw, qtype), raw)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return str(path), want


def test_metadata_round_trip(tiny_gguf):
    path, _ = tiny_gguf
    f = gj.load_gguf(path, device="cpu")
    assert f.metadata["general.architecture"] == "llama"
    assert f.metadata["general.name"] == "tiny test model"
    assert f.metadata["test.some_number"] == 42
    assert f.metadata["test.some_float"] == 0.5
    assert list(f.metadata["test.some_list"]) == [1, 2, 3]
    assert "6 tensors" in repr(f)


def test_payloads_shapes_and_qtypes_on_the_host(tiny_gguf):
    path, want = tiny_gguf
    f = gj.load_gguf(path, dtype=torch.float32, device="cpu")
    assert set(f.tensors) == set(want)
    for name, (qtype, dense, raw) in want.items():
        qa = f.tensors[name]
        assert qa.qtype == qtype and qa.shape == dense.shape and qa.dtype == torch.float32, name
        assert qa.data.dtype == torch.uint8, name
        bs, ts = GGML_QUANT_SIZES[qtype]
        assert tuple(qa.data.shape) == (*dense.shape[:-1], dense.shape[-1] // bs * ts), name
        # the stored bytes are the file's bytes, untouched
        assert np.array_equal(qa.data.numpy().reshape(-1), np.ascontiguousarray(raw).reshape(-1)), name
        # and the CPU checker decodes them to what gguf-py says
        O.assert_bitwise_equal(O.c_dequantize(qa.data.numpy().reshape(-1, qa.data.shape[-1]), qtype).reshape(dense.shape),
                               np.asarray(dense, dtype=np.float32), name)


def test_tensor_filter(tiny_gguf):
    path, _ = tiny_gguf
    f = gj.load_gguf(path, tensor_filter=lambda name: "ffn" in name, device="cpu")
    assert set(f.tensors) == {"blk.0.ffn_up.weight", "blk.0.ffn_down.weight"}


def test_row_sharded_load_takes_a_contiguous_byte_range(tiny_gguf):
    path, want = tiny_gguf
    whole = gj.load_gguf(path, device="cpu").tensors
    for rank in range(4):
        part = gj.load_gguf(path, device="cpu", shard=(rank, 4)).tensors
        for name, (qtype, dense, _) in want.items():
            if dense.ndim == 2 and dense.shape[0] % 4 == 0:
                rows = dense.shape[0] // 4
                assert part[name].shape == (rows, dense.shape[1]), name
                assert torch.equal(part[name].data, whole[name].data[rank * rows:(rank + 1) * rows]), name
            else:
                assert part[name].shape == whole[name].shape and torch.equal(part[name].data, whole[name].data), name


def test_default_dtype_is_bf16(tiny_gguf):
    path, _ = tiny_gguf
    f = gj.load_gguf(path, device="cpu")
    assert all(qa.dtype == torch.bfloat16 for qa in f.tensors.values())


def test_host_resident_arrays_refuse_to_decode(tiny_gguf):
    path, _ = tiny_gguf
    f = gj.load_gguf(path, device="cpu")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        f.tensors["blk.0.attn_q.weight"].dequantize()


@pytest.mark.gpu
def test_loaded_tensors_decode_bitwise_on_the_device(tiny_gguf):
    path, want = tiny_gguf
    f = gj.load_gguf(path, dtype=torch.float32)
    assert set(f.tensors) == set(want)
    for name, (qtype, dense, _) in want.items():
        qa = f.tensors[name]
        assert qa.data.is_cuda and qa.shape == dense.shape, name
        out = qa.dequantize()
        assert out.dtype == torch.float32 and tuple(out.shape) == dense.shape
        O.assert_bitwise_equal(out.cpu().numpy(), np.asarray(dense, dtype=np.float32), name)
    half = gj.load_gguf(path).tensors["blk.0.attn_q.weight"].dequantize()
    assert half.dtype == torch.bfloat16
