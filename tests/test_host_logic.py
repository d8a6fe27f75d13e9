"""Host-side logic that needs no GPU: definitions, signatures, the kernel registry, Buffer, the
CompiledKernel argument checks (against a recording stand-in for the C function), the exported C ABI,
and row sharding over two gloo ranks."""
from __future__ import annotations

import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


# ------------------------------------------------------------------ definitions and registry

def test_package_surface_matches_the_reference_names():
    import weft_b200 as weft
    from weft_b200 import runtime

    for name in ["DefinitionError", "DerivedEncodingDefinition", "EncodingDefinition", "FrontendError", "KernelDefinition",
                 "LanguageUseError", "WeftError", "derive", "compile", "encoding", "kernel", "jit", "lower_to_mlir", "overloads"]:
        assert hasattr(weft, name), name
    for name in ["Buffer", "CompilationError", "CompiledKernel", "CompileOptions", "JITKernel", "NativeTarget", "Toolchain",
                 "compile", "jit"]:
        assert hasattr(runtime, name), name


def test_definitions_are_inert():
    import weft_b200 as weft
    import weft_b200.language as wl
    from weft_b200.kernels import vec_dot

    with pytest.raises(weft.LanguageUseError):
        vec_dot.quantized_vec_dot_q4_k_q8_k(None, None, None)
    with pytest.raises(weft.LanguageUseError):
        wl.load(1)
    with pytest.raises(weft.LanguageUseError):
        wl.f32(1.0)
    with pytest.raises(weft.DefinitionError):
        weft.kernel(42)
    assert "quantized_vec_dot_q4_k_q8_k" in repr(vec_dot.quantized_vec_dot_q4_k_q8_k)


def test_record_geometry_comes_out_of_the_declarations():
    from weft_b200 import formats
    from weft_b200.signature import encoding_facts

    for name, facts in formats.RECORDS.items():
        assert encoding_facts(getattr(formats, name)) == facts
    assert formats.row_bytes("Q4_K", 4096) == 2304 and formats.row_bytes("Q8_K", 4096) == 4672
    with pytest.raises(ValueError):
        formats.row_bytes("Q4_K", 100)


def test_kernel_abi_follows_the_reference_rules():
    from weft_b200 import registry
    from weft_b200.kernels import dequantize, mul_mat

    abi = registry.resolve(mul_mat.production_mul_mat_iq2_xxs_decode)
    assert [a["name"] for a in abi["arguments"]] == ["W", "X", "Xq", "grid", "signs", "Y"]
    assert [a["alias_set"] for a in abi["arguments"]] == [0, 0, 1, 0, 0, 2]          # named groups numbered by first appearance
    assert [a["writable"] for a in abi["arguments"]] == [False, False, True, False, False, True]
    assert abi["shape_parameters"] == ["N", "K", "M"] and abi["c_dimension_order"] == ["N", "K", "M"]
    w, x = abi["arguments"][0], abi["arguments"][1]
    assert (w["encoding"], w["storage_bytes"], w["record_elements"], w["alignment"]) == ("IQ2_XXS", 66, 256, 2)
    assert (x["encoding"], x["storage_bytes"], x["record_elements"], x["alignment"], x["c_type"]) == ("dense.f32", 4, 1, 4, "float")
    deq = registry.resolve(dequantize.row_dequantize_tq1_0)
    assert [a["encoding"] for a in deq["arguments"]] == ["TQ1_0", "dense.u32", "dense.f32"]
    assert deq["arguments"][1]["shape"] == ["5"] and deq["shape_parameters"] == ["K"]
    assert len(registry.supported_symbols()) == 105


_EXTRA_KERNELS = """
from __future__ import annotations
import weft_b200 as weft
import weft_b200.language as wl
from weft_b200 import formats as ggml

@weft.kernel
def gemm_f32(A: wl.View[wl.f32, (M, K)], B: wl.View[wl.f32, (K, N)], C: wl.View[wl.f32, (M, N)]): ...

@weft.kernel
def row_dequantize_q4_k(W: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (K,)]): ...

@weft.kernel
def row_dequantize_q4_0(W: wl.View[ggml.Q4_0, (K,)], Y: wl.View[wl.f32, (J,)]): ...

@weft.kernel
def row_dequantize_q8_0(W: wl.View[ggml.Q8_0, (COLS,)], Y: wl.View[wl.f32, (COLS,)]): ...
"""


def test_registry_refuses_what_it_cannot_run(tmp_path):
    import importlib.util

    import weft_b200 as weft
    from weft_b200 import registry

    path = tmp_path / "extra_kernels.py"
    path.write_text(_EXTRA_KERNELS)
    spec = importlib.util.spec_from_file_location("extra_kernels", path)
    extra = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(extra)
    with pytest.raises(NotImplementedError):
        registry.resolve(extra.gemm_f32)                      # no generic lowering, no fallback
    with pytest.raises(TypeError):
        registry.resolve(extra.row_dequantize_q4_k)           # wrong Encoding for this symbol
    with pytest.raises(TypeError):
        registry.resolve(extra.row_dequantize_q4_0)           # extents that the kernel ties together are untied
    # the same signature under other symbol names is the same kernel
    assert registry.resolve(extra.row_dequantize_q8_0)["c_dimension_order"] == ["COLS"]
    with pytest.raises(weft.DefinitionError):                 # a definition without inspectable source, as in the reference
        exec("import weft_b200 as weft\n@weft.kernel\ndef f(): ...", {})


def test_reference_kernel_files_resolve_unchanged():
    """The reference's own kernel files import against this package and map onto the same C symbols."""
    root = os.environ.get("WEFT_REFERENCE_ROOT")
    examples = Path(root) / "examples" if root else ROOT.parent / "reference" / "examples"
    if not examples.exists():
        pytest.skip("reference tree not present (WEFT_REFERENCE_ROOT, or a checkout named reference beside this repository)")
    code = (
        "import sys; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "import weft_b200; weft_b200.install_as_weft()\n"
        "from weft_b200 import registry\n"
        "import kernels.mul_mat.q4_k_decode as a, kernels.mul_mat.q4_k_staged as b, kernels.dequantize.iq2_xxs as c, kernels.vec_dot.tq1_0_q8_k as d, kernels.quantize.q8_k as e\n"
        "r = registry.resolve(a.production_mul_mat_q4_k_decode); assert [x['alias_set'] for x in r['arguments']] == [0, 0, 1, 2], r\n"
        "assert registry.resolve(b.production_mul_mat_q4_k_staged)['c_dimension_order'] == ['N', 'K', 'M']\n"
        "assert [x['alias_set'] for x in registry.resolve(c.row_dequantize_iq2_xxs)['arguments']] == [0, 0, 0, 1]\n"
        "assert registry.resolve(d.quantized_vec_dot_tq1_0_q8_k)['shape_parameters'] == ['K']\n"
        "assert registry.resolve(e.q8_K_quantize)['arguments'][1]['encoding'] == 'Q8_K'\n"
        "import kernels.gemv.q4_k as f, kernels.mul_mat.q4_k_persistent as g\n"
        "r = registry.resolve(f.q4_k_q8_k_gemv); assert r['arguments'][0]['encoding'] == 'Q4K_I[16]' and r['c_dimension_order'] == ['M', 'K'], r\n"
        "r = registry.resolve(g.production_mul_mat_q4_k_persistent); assert (r['arguments'][0]['storage_bytes'], r['arguments'][0]['record_elements']) == (144, 256)\n"
        "assert r['shape_parameters'] == ['N', 'K', 'M'] and r['c_dimension_order'] == ['M', 'K', 'N'], r\n"
        "import kernels.gemv.q4_k_groups4 as h, kernels.gemv.q4_k_contract as i, kernels.vec_dot.tq1_0_q8_k_lane16 as j\n"
        "import kernels.mul_mat.tq1_0_lane16_decode as k, kernels.mul_mat.q3_k_predecoded_scales_decode as l, kernels.mul_mat.q3_k_predecoded_scales as m\n"
        "assert registry.resolve(h.q4_k_q8_k_gemv_groups4)['c_dimension_order'] == ['M', 'K']\n"
        "assert registry.resolve(i.q4_k_q8_k_gemv_contract)['arguments'][0]['encoding'] == 'Q4K_I[16]'\n"
        "assert [x['name'] for x in registry.resolve(j.quantized_vec_dot_tq1_0_q8_k_lane16)['arguments']] == ['W', 'X', 'powers', 'Y']\n"
        "assert [x['alias_set'] for x in registry.resolve(k.production_mul_mat_tq1_0_lane16_decode)['arguments']] == [0, 0, 1, 0, 2]\n"
        "assert registry.resolve(l.production_mul_mat_q3_k_predecoded_scales_decode)['c_dimension_order'] == ['N', 'K', 'M']\n"
        "assert registry.resolve(m.production_mul_mat_q3_k_predecoded_scales)['c_dimension_order'] == ['N', 'K', 'M']\n"
        "print('ok')\n" % (str(ROOT), str(examples)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"})
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr


def test_derived_encoding_keeps_its_base_record_geometry():
    """Q4K_I[16] is Q4_K records, 16 rows interleaved: same storage per record, same alignment (Emitter.h:321-333);
    the persistent kernel's C symbol takes its extents as (M, K, N) (mul_mat_runtime.cpp:337-348)."""
    from weft_b200 import registry
    from weft_b200.kernels import gemv, mul_mat

    abi = registry.resolve(gemv.q4_k_q8_k_gemv)
    w = abi["arguments"][0]
    assert (w["encoding"], w["storage_bytes"], w["record_elements"], w["alignment"]) == ("Q4K_I[16]", 144, 256, 2)
    assert abi["shape_parameters"] == ["M", "K"] and [a["access"] for a in abi["arguments"]] == ["read", "read", "write"]
    abi = registry.resolve(mul_mat.production_mul_mat_q4_k_persistent)
    assert abi["shape_parameters"] == ["N", "K", "M"] and abi["c_dimension_order"] == ["M", "K", "N"]


# ------------------------------------------------------------------ Buffer and the call checks

def test_buffer_borrows_and_infers():
    from weft_b200.runtime import Buffer

    a = np.zeros((3, 8), dtype=np.float32)
    b = Buffer(a)
    assert (b.shape, b.encoding, b.nbytes, b.readonly, b.device) == ((3, 8), "dense.f32", 96, False, None)
    assert b.address == a.ctypes.data
    packed = np.zeros(144 * 4, dtype=np.uint8)
    q = Buffer(packed, shape=(1, 1024), encoding="Q4_K")
    assert q.shape == (1, 1024) and q.encoding == "Q4_K" and q.nbytes == 576
    with pytest.raises(ValueError):
        Buffer(np.zeros((4, 4), dtype=np.float32)[:, ::2])
    with pytest.raises(ValueError):
        Buffer(packed, shape=(1, -4), encoding="Q4_K")
    with pytest.raises(TypeError):
        Buffer(np.zeros(2, dtype=[("a", np.int8), ("b", np.int16)]))
    assert Buffer(bytes(16)).readonly
    torch = pytest.importorskip("torch")
    t = torch.zeros((2, 5), dtype=torch.int8)
    tb = Buffer(t)
    assert (tb.shape, tb.encoding, tb.address, tb.device) == ((2, 5), "dense.i8", t.data_ptr(), None)


class _Recorder:
    def __init__(self):
        self.calls = []
        self.argtypes = None
        self.restype = None

    def __call__(self, *args):
        self.calls.append(args)
        return 0


def _compiled(definition):
    """A CompiledKernel in front of a recording stand-in: exercises every host-side check without a GPU."""
    from weft_b200 import registry
    from weft_b200.runtime.compiler import ARTIFACT_KIND, CompiledKernel, CompileOptions
    from weft_b200.runtime.driver import NativeTarget

    target = NativeTarget(march="sm_100a", abi="weft_b200-c", xlen=64, vlen_bits=1024, cpus=frozenset({0}), library="")
    kernel = registry.resolve(definition)
    kernel.update({"march": target.march, "abi": target.abi, "vlen_bits": target.vlen_bits, "bindings": {}})
    artifact = {"kind": ARTIFACT_KIND, "riscv_ir": "", "intrinsic_c": "", "kernels": [kernel]}
    compiled = CompiledKernel.__new__(CompiledKernel)
    import threading
    from weft_b200.runtime.compiler import _freeze

    compiled.metadata = _freeze(kernel)
    compiled.target, compiled.options = target, CompileOptions()
    compiled._lock, compiled._signature = threading.RLock(), definition.signature
    compiled._library, compiled._function, compiled.closed = None, _Recorder(), False
    assert artifact["kind"]
    return compiled


def test_call_checks_in_reference_order():
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    k = _compiled(mul_mat.production_mul_mat_q4_k_decode)
    n, kk, m = 4, 512, 2
    w = Buffer(np.zeros(n * 288, dtype=np.uint8), shape=(n, kk), encoding="Q4_K")
    x = np.zeros((m, kk), dtype=np.float32)
    xq = Buffer(np.zeros(m * 584, dtype=np.uint8), shape=(m, kk), encoding="Q8_K")
    y = np.zeros((m, n), dtype=np.float32)
    k(w, x, xq, y)
    args = k._function.calls[-1]
    assert args[:4] == (w.address, x.ctypes.data, xq.address, y.ctypes.data) and args[4:] == (n, kk, m)
    k(W=w, X=x, Xq=xq, Y=y)                                            # keywords bind like the Python signature
    with pytest.raises(TypeError, match="requires Q8_K"):
        k(w, x, Buffer(np.zeros(m * 584, dtype=np.uint8), shape=(m, kk), encoding="Q8_0"), y)
    with pytest.raises(ValueError, match="rank"):
        k(w, x[0], xq, y)
    with pytest.raises(ValueError, match="disagrees with extent K"):
        k(w, np.zeros((m, 256), dtype=np.float32), xq, y)
    with pytest.raises(ValueError, match="complete Encoding records"):
        k(Buffer(np.zeros(n * 288, dtype=np.uint8), shape=(n, 500), encoding="Q4_K"), np.zeros((m, 500), dtype=np.float32), xq, y)
    with pytest.raises(ValueError, match="shorter"):
        k(Buffer(np.zeros(100, dtype=np.uint8), shape=(n, kk), encoding="Q4_K"), x, xq, y)
    with pytest.raises(TypeError, match="writable"):
        k(w, x, xq, Buffer(bytes(m * n * 4), shape=(m, n), encoding="dense.f32"))
    shared = np.zeros(m * 584 + 64, dtype=np.uint8)
    with pytest.raises(ValueError, match="aliases"):                     # Xq and Y are in different alias groups
        k(w, x, Buffer(shared[: m * 584], shape=(m, kk), encoding="Q8_K"), Buffer(shared[:32].view(np.float32), shape=(m, n)))
    with pytest.raises(ValueError, match="alignment"):
        k(w, x, Buffer(np.zeros(m * 584 + 8, dtype=np.uint8)[2:2 + m * 584], shape=(m, kk), encoding="Q8_K"), y)
    k.close(); k.close()
    with pytest.raises(RuntimeError):
        k(w, x, xq, y)


def test_compile_options_keep_the_reference_record():
    from weft_b200.runtime import CompileOptions

    o = CompileOptions(meta={"NC": 64, "KC": 512})
    assert o.arguments()[:2] == ["--meta=KC=512", "--meta=NC=64"] and "--matrix-extension=none" in o.arguments()
    with pytest.raises(ValueError):
        CompileOptions(meta={"NC": 0})
    with pytest.raises(ValueError):
        CompileOptions(meta={"not an identifier": 4})


# ------------------------------------------------------------------ the C ABI library

def _declared_symbols():
    header = (ROOT / "include" / "weft_b200.h").read_text()
    return sorted(set(re.findall(r"^(?:int|size_t|const char \*|unsigned long long)\s*\*?\s*(\w+)\(", header, flags=re.M)))


def test_library_exports_every_declared_symbol():
    from weft_b200 import build

    library = build.ensure_built()
    lib = ctypes.CDLL(str(library))
    names = _declared_symbols()
    assert len(names) >= 50 and "production_mul_mat_q4_k_decode" in names and "weft_b200_mul_mat_shard" in names
    assert "q4_k_q8_k_gemv_W_packed_size" in names and "production_mul_mat_q4_k_persistent_W_pack" in names
    for name in names:
        assert hasattr(lib, name), name


def test_library_fails_loudly_without_a_gpu():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from weft_b200 import build

    lib = ctypes.CDLL(str(build.ensure_built()))
    lib.weft_b200_last_error.restype = ctypes.c_char_p
    y = np.zeros(256, dtype=np.float32)
    w = np.zeros(144, dtype=np.uint8)
    lib.row_dequantize_q4_k.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    assert lib.row_dequantize_q4_k(w.ctypes.data, y.ctypes.data, 256) != 0      # no CPU fallback
    assert b"no CUDA device" in lib.weft_b200_last_error()
    import weft_b200 as weft
    from weft_b200.kernels import rows
    from weft_b200.runtime import CompilationError

    with pytest.raises(CompilationError):
        weft.compile(rows.row_dequantize_q4_k_rows)


# ------------------------------------------------------------------ row sharding

def test_shard_plan_covers_rows_once():
    from weft_b200 import sharding

    for n, world in [(14336, 8), (28672, 8), (4096, 4), (10, 4), (3, 8)]:
        plans = sharding.plan(n, 4096, "Q4_K", world)
        assert plans[0].begin == 0 and plans[-1].end == n
        assert all(a.end == b.begin for a, b in zip(plans, plans[1:]))
        assert max(p.rows for p in plans) - min(p.rows for p in plans) <= 1
    s = sharding.shard_of(14336, 4096, "Q4_K", 3, 8)
    assert s.byte_range == (3 * 1792 * 2304, 4 * 1792 * 2304)
    with pytest.raises(ValueError):
        sharding.shard_of(8, 4096, "Q4_K", 8, 8)


_WORKER = r"""
import os, sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch, torch.distributed as dist
import oracle
from weft_b200 import sharding
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
n, k, m = 90, 512, 3                        # 90 rows over 2 ranks; also exercised with an uneven split below
rng = np.random.default_rng(11)
w = oracle.quantize(oracle.Q4_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
x = rng.standard_normal((m, k)).astype(np.float32)
full, _ = oracle.mul_mat(oracle.Q4_K, w, x, n, k, m, rule=1)
for rows in (n, n - 1):
    shard = sharding.shard_of(rows, k, "Q4_K", rank, world)
    lo, hi = shard.byte_range
    local_w = w.reshape(-1)[lo:hi]
    def local(y_local):                      # the CPU oracle stands in for the GPU kernel in this host-logic test
        part, _ = oracle.mul_mat(oracle.Q4_K, local_w, x, shard.rows, k, m, rule=1)
        y_local.copy_(torch.from_numpy(part))
    y = sharding.sharded_mul_mat(shard, m, local)
    assert tuple(y.shape) == (m, rows)
    assert np.array_equal(y.numpy().view(np.uint32), full[:, :rows].view(np.uint32)), "sharded result differs"

# peer buffer tables: a stand-in for the C library hands out rank-tagged "device pointers" and handles
from weft_b200 import peers
class Fn:
    def __init__(self, call): self.call, self.argtypes = call, None
    def __call__(self, *a): return self.call(*a)
class FakeLib:
    def __init__(self):
        self.count, self.closed, self.freed = 0, [], []
        self.weft_b200_peer_alloc, self.weft_b200_peer_open = Fn(self.alloc), Fn(self.open)
        self.weft_b200_peer_close, self.weft_b200_peer_free = Fn(lambda p: self.closed.append(p.value) or 0), Fn(lambda p: self.freed.append(p.value) or 0)
    def alloc(self, size, slot, handle):
        self.count += 1
        slot._obj.value = 0x100000 * (rank + 1) + 0x100 * self.count
        handle.raw = (b"rank%d-buffer%d-size%d" % (rank, self.count, size)).ljust(64, b".")
        return 0
    def open(self, handle, slot):
        owner, index = int(handle[4:5]), int(handle.split(b"-")[1][6:])
        slot._obj.value = 0x900000 + 0x100000 * (owner + 1) + 0x100 * index      # a different mapping of the owner's buffer
        return 0
fake = FakeLib()
group = peers.PeerBuffers(fake, world, rank, [4096, 4096, 4 * peers.SYNC_INTS])
assert len(group.tables) == 3 and all(len(t) == world for t in group.tables)
for index, table in enumerate(group.tables):
    for peer in range(world):
        want = (0x100000 * (rank + 1) if peer == rank else 0x900000 + 0x100000 * (peer + 1)) + 0x100 * (index + 1)
        assert table[peer] == want, (index, peer, hex(table[peer] or 0))
order = []
group.close(lambda: (order.append(len(fake.closed)), dist.barrier()))
assert order == [3 * (world - 1)] and len(fake.freed) == 3 and not fake.closed[0] in fake.freed
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_sharded_mul_mat_two_gloo_ranks(tmp_path, oracle):
    pytest.importorskip("torch")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = {**os.environ, "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29731", "WORLD_SIZE": "2"}
    procs = [subprocess.Popen([sys.executable, str(script), str(ROOT)], env={**env, "RANK": str(r)},
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    for r, proc in enumerate(procs):
        out, err = proc.communicate(timeout=240)
        assert proc.returncode == 0 and f"rank {r} ok" in out, err[-2000:]
