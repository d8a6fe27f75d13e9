"""Run under torchrun on N >= 2 GPUs of one node (tests/test_gpu_multi.py does that): the row-sharded mul_mat
whose all-gather is done by the library's own kernels over peer memory, against the CPU oracle on every rank."""
from __future__ import annotations

import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from helpers import TQ1_POWERS, activations, rel_l2, weights  # noqa: E402
from weft_b200.formats import FORMAT_IDS, row_bytes  # noqa: E402
from weft_b200.peers import STAGE_BYTES, SYNC_INTS, PeerBuffers  # noqa: E402
from weft_b200.runtime.driver import Toolchain, last_error, load_library  # noqa: E402

CASES = [
    # (format, mode, N, K, M): fused peer stores in the ring GEMVs, push kernel behind the others
    ("Q4_K", 0, 4096, 4096, 1),
    ("Q4_K", 0, 1000, 2048, 3),      # uneven row blocks, several activation rows
    ("Q6_K", 0, 2048, 2048, 2),
    ("Q4_0", 0, 1024, 4096, 1),
    ("TQ1_0", 0, 512, 1024, 1),      # rows of 216 bytes: fallback GEMV + push kernel
    ("Q4_K", 1, 1024, 2048, 128),    # tensor-core prefill + push kernel
    ("TQ1_0", 1, 640, 2048, 300),    # CTA-pair prefill on activation planes + push kernel
]


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")          # handles travel as Python objects; no collective library touches the data
    lib = load_library(Toolchain().resolve().compiler)
    if lib.weft_b200_init(local):
        raise SystemExit(last_error(lib))
    fn = lib.weft_b200_mul_mat_shard_gather
    fn.argtypes = ([ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 6 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
                   + [ctypes.c_size_t] * 5 + [ctypes.c_uint])
    lib.weft_b200_peer_read.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    golden = np.load(ROOT / "tests" / "golden" / "golden.npz")
    grid, signs = golden["iq2xxs_grid"], golden["iq2xxs_signs"]
    grid_dev, signs_dev = torch.from_numpy(grid).cuda(), torch.from_numpy(signs).cuda()
    powers_dev = torch.from_numpy(TQ1_POWERS.view(np.int32)).cuda()
    # One set of buffers for every case: calls of different shapes follow each other on the same outputs, sync
    # blocks and staging area (a layer's projections do), and the epochs run on across them.
    largest = max(m * n for _, _, n, _, m in CASES)
    peers = PeerBuffers(lib, world, rank, [4 * largest, 4 * largest, 4 * SYNC_INTS, STAGE_BYTES])
    calls = 0
    for fmt, mode, n, k, m in CASES:
        fid = oracle.FORMAT_IDS[fmt]
        rng = np.random.default_rng(n + k + m)          # same inputs on every rank
        w = weights(fid, rng, n, k)
        x = activations(rng, m, k)
        want, _ = oracle.mul_mat(fid, w, x, n, k, m, rule=1, grid=grid, signs=signs)
        n0, n1 = n * rank // world, n * (rank + 1) // world
        w_dev = torch.from_numpy(np.ascontiguousarray(w[n0:n1])).cuda()
        x_dev = torch.from_numpy(x).cuda()
        act = "Q8_0" if fmt in ("Q4_0", "Q8_0") else "Q8_K"
        xq_dev = torch.zeros((m, row_bytes(act, k)), dtype=torch.uint8, device="cuda")
        for step in range(3):                            # several epochs, alternating output buffers (odd count: the next case starts on the other half)
            out = calls % 2
            calls += 1
            status = fn(FORMAT_IDS[fmt], mode, w_dev.data_ptr(), x_dev.data_ptr(), xq_dev.data_ptr(), grid_dev.data_ptr(), signs_dev.data_ptr(),
                        powers_dev.data_ptr(), peers.tables[out], peers.tables[2], peers.tables[3], world, rank, n0, n1 - n0, n, k, m, 0)
            if status:
                raise SystemExit(f"rank {rank} {fmt} step {step}: " + last_error(lib))
            got = np.empty((m, n), dtype=np.float32)
            if lib.weft_b200_peer_read(got.ctypes.data, peers.local[out], got.nbytes):
                raise SystemExit(f"rank {rank} {fmt} step {step}: " + last_error(lib))
            error = rel_l2(got, want)
            if not error <= 1e-5:
                raise SystemExit(f"rank {rank}: {fmt} mode {mode} ({n}, {k}, {m}) step {step}: relative L2 {error}")
        torch.cuda.synchronize()
        dist.barrier()                                   # every rank has read this case's outputs before the next case overwrites them
    peers.close(dist.barrier)
    dist.barrier()
    if rank == 0:
        print(f"multi_gpu_gather ok: {len(CASES)} cases on {world} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
