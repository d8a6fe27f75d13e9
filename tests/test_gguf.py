"""GGUF tensors -> Buffers: the file reader on CPU, and a mapped tensor through the decode kernel on the GPU."""
from __future__ import annotations

import struct

import numpy as np
import pytest

from helpers import activations, rel_l2, weights


def _model(oracle, rng):
    n, k = 96, 1024
    return {
        "blk.0.attn_q.weight": ("Q4_K", (n, k), weights(oracle.Q4_K, rng, n, k)),
        "blk.0.ffn_down.weight": ("Q6_K", (64, 512), weights(oracle.Q6_K, rng, 64, 512)),
        "blk.0.attn_k.weight": ("Q8_0", (32, 256), weights(oracle.Q8_0, rng, 32, 256)),
        "blk.0.attn_norm.weight": ("dense.f32", (k,), rng.standard_normal(k).astype(np.float32)),
    }


def test_gguf_round_trip(tmp_path, oracle):
    from weft_b200 import gguf

    rng = np.random.default_rng(4)
    tensors = _model(oracle, rng)
    path = tmp_path / "model.gguf"
    gguf.write(path, tensors, {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 10000.0,
                               "tokenizer.ggml.tokens": ["<s>", "a"], "general.quantized": True})
    with gguf.read(path) as model:
        assert model.version == 3 and model.metadata["general.architecture"] == "llama"
        assert model.metadata["llama.block_count"] == 1 and model.metadata["tokenizer.ggml.tokens"] == ["<s>", "a"]
        assert list(model.tensors) == list(tensors)
        for name, (encoding, shape, data) in tensors.items():
            info = model.tensors[name]
            assert info.encoding == encoding and info.shape == tuple(shape) and info.offset % 32 == 0
            assert np.array_equal(model.raw(name), np.ascontiguousarray(data).reshape(-1).view(np.uint8))
            buffer = model.buffer(name)
            assert buffer.encoding == encoding and tuple(buffer.shape) == tuple(shape) and buffer.device is None
        # the mapped records dequantize like the originals
        q = model.tensors["blk.0.attn_q.weight"]
        got = oracle.dequantize(oracle.Q4_K, np.array(model.raw(q.name)).reshape(q.shape[0], -1), q.shape[1])
        assert np.array_equal(got, oracle.dequantize(oracle.Q4_K, tensors[q.name][2], q.shape[1]))
    # another alignment, and the errors a damaged file must raise
    gguf.write(tmp_path / "a64.gguf", tensors, alignment=64)
    with gguf.read(tmp_path / "a64.gguf") as model:
        assert all(info.offset % 64 == 0 for info in model.tensors.values())
    (tmp_path / "bad.gguf").write_bytes(b"GGML" + bytes(60))
    with pytest.raises(ValueError):
        gguf.read(tmp_path / "bad.gguf")
    whole = path.read_bytes()
    (tmp_path / "short.gguf").write_bytes(whole[:-100])
    with pytest.raises(ValueError):
        gguf.read(tmp_path / "short.gguf")
    (tmp_path / "v9.gguf").write_bytes(whole[:4] + struct.pack("<I", 9) + whole[8:])
    with pytest.raises(NotImplementedError):
        gguf.read(tmp_path / "v9.gguf")
    with pytest.raises(ValueError):
        gguf.write(tmp_path / "odd.gguf", {"w": ("Q4_K", (2, 1000), np.zeros(10, dtype=np.uint8))})


@pytest.mark.gpu
def test_gguf_tensor_through_the_decode_kernel(tmp_path, oracle):
    import torch

    import weft_b200 as weft
    from weft_b200 import gguf
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    rng = np.random.default_rng(8)
    n, k = 512, 2048
    w = weights(oracle.Q4_K, rng, n, k)
    gguf.write(tmp_path / "layer.gguf", {"blk.0.ffn_up.weight": ("Q4_K", (n, k), w)})
    x = activations(rng, 1, k)
    want, _ = oracle.mul_mat(oracle.Q4_K, w, x, n, k, 1, rule=1)
    kernel = weft.compile(mul_mat.production_mul_mat_q4_k_decode)
    with gguf.read(tmp_path / "layer.gguf") as model:
        for device in (None, "cuda"):          # host mapping (staged by the C ABI) and a device copy
            xq = torch.zeros((1, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
            y = torch.empty((1, n), device="cuda")
            kernel(model.buffer("blk.0.ffn_up.weight", device=device), torch.from_numpy(x).cuda(), Buffer(xq, shape=(1, k), encoding="Q8_K"), y)
            assert rel_l2(y.cpu().numpy(), want) <= 1e-5


@pytest.mark.gpu
def test_llama_block_projection_chain(tmp_path, oracle):
    """A small Llama-shaped block from a GGUF file (Q4_K projections, Q6_K ffn_down as in Q4_K_M models) through
    weft_b200_mul_mat_chain, every projection against the oracle; the chain also replays from a CUDA graph."""
    import ctypes

    import torch

    from weft_b200 import gguf
    from weft_b200.formats import row_bytes
    from weft_b200.layers import Projection, ProjectionChain, llama_block_steps
    from weft_b200.runtime.driver import Toolchain, load_library

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    lib = load_library(Toolchain().resolve().compiler)
    rng = np.random.default_rng(21)
    hidden, kv, ffn = 1024, 256, 2048
    dims = {"attn_q": (hidden, hidden), "attn_k": (kv, hidden), "attn_v": (kv, hidden), "attn_output": (hidden, hidden),
            "ffn_gate": (ffn, hidden), "ffn_up": (ffn, hidden), "ffn_down": (hidden, ffn)}
    packed = {}
    for part, (n, k) in dims.items():
        encoding = "Q6_K" if part == "ffn_down" else "Q4_K"
        packed[f"blk.0.{part}.weight"] = (encoding, (n, k), weights(oracle.FORMAT_IDS[encoding], rng, n, k))
    gguf.write(tmp_path / "block.gguf", packed, {"general.architecture": "llama"})
    source = {"attn_q": "h", "attn_k": "h", "attn_v": "h", "attn_output": "a", "ffn_gate": "g", "ffn_up": "g", "ffn_down": "f"}
    x = {key: activations(rng, 1, k) for key, k in (("h", hidden), ("a", hidden), ("g", hidden), ("f", ffn))}
    x_dev = {key: torch.from_numpy(v).cuda() for key, v in x.items()}
    xq_dev = {key: torch.zeros((1, row_bytes("Q8_K", v.shape[1])), dtype=torch.uint8, device="cuda") for key, v in x.items()}
    with gguf.read(tmp_path / "block.gguf") as model:
        steps = llama_block_steps(model, 0)
        w_dev = {name: torch.from_numpy(np.array(model.raw(name))).cuda() for name, _, _, _ in steps}
    y_dev, projections, seen = {}, [], set()
    for name, encoding, n, k in steps:
        part = name.split(".")[2]
        key = source[part]
        y_dev[name] = torch.full((1, n), float("nan"), device="cuda")
        projections.append(Projection(encoding, w_dev[name].data_ptr(), x_dev[key].data_ptr(), xq_dev[key].data_ptr(), y_dev[name].data_ptr(),
                                      n, k, reuse_xq=key in seen))
        seen.add(key)
    chain = ProjectionChain(lib, projections)
    assert chain.weight_bytes == sum(w.numel() for w in w_dev.values())
    chain.run()
    assert lib.weft_b200_synchronize() == 0

    def check_all():
        for name, encoding, n, k in steps:
            want, _ = oracle.mul_mat(oracle.FORMAT_IDS[encoding], packed[name][2], x[source[name.split(".")[2]]], n, k, 1, rule=1)
            assert rel_l2(y_dev[name].cpu().numpy(), want) <= 1e-5, name

    check_all()
    # replay from a CUDA graph on a caller-owned stream
    for y in y_dev.values():
        y.fill_(float("nan"))
    side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    lib.weft_b200_set_stream(ctypes.c_void_p(side.cuda_stream))
    lib.weft_b200_set_async(1)
    try:
        with torch.cuda.graph(graph, stream=side):
            chain.run()
    finally:
        lib.weft_b200_set_stream(None)
        lib.weft_b200_set_async(0)
    graph.replay()
    torch.cuda.synchronize()
    check_all()
    # a bad step is reported, not executed
    broken = ProjectionChain(lib, [Projection("Q4_K", 0, 0, 0, 0, 16, 100)])
    with pytest.raises(RuntimeError):
        broken.run()
