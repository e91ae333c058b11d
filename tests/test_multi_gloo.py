"""The N > 1 path on CPU ranks (gloo, world size 2 and 3): shard planning, per-rank conversion
and the all-gather of the row-sharded C.  The device kernel is replaced by the CPU oracle here;
what is under test is the host logic every rank runs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import hopper_spmm_b200 as hs
        import oracle
        from hopper_spmm_b200 import sharded, synth
        csr, B = synth.make_config("rmat24_sharded_fp16", 0, "cpu", 12)  # every rank generates the same inputs
        rp, ci, v = csr.numpy()
        cuts, r0, r1 = sharded.my_rows(csr.rows, rp, world, rank)
        prp, pci, pv = sharded.slice_csr(rp, ci, v, r0, r1)
        part = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(r1 - r0, csr.cols, prp, pci, pv))
        # this rank's slice of the whole-matrix format
        whole = hs.CSR2BTCFNOBITMAP(hs.CSR_MTX(csr.rows, csr.cols, rp, ci, v))
        mine = (np.asarray(whole.rowIdx) >= r0) & (np.asarray(whole.rowIdx) < r1)
        assert np.array_equal(np.asarray(part.rowIdx) + r0, np.asarray(whole.rowIdx)[mine])
        t0 = int(np.asarray(whole.rowOffset)[np.argmax(mine)]) if mine.any() else 0
        assert np.array_equal(part.tcA2B, whole.tcA2B[t0 * 16:(t0 + part.total_tiles) * 16])
        assert np.array_equal(np.asarray(part.data).view(np.uint16),
                              np.asarray(whole.data).view(np.uint16)[t0 * 256:(t0 + part.total_tiles) * 256])
        # local product (oracle stands in for the device), then the collective
        C_local = torch.from_numpy(oracle.spmm_csr(r1 - r0, prp, pci, pv, B.numpy()))
        full = sharded.allgather_rows(C_local, cuts)
        want = oracle.spmm_csr(csr.rows, rp, ci, v, B.numpy())
        assert np.array_equal(full.numpy(), want)  # same per-row order of additions: bit-identical
        # the exchange itself on crafted cuts: equal slices, skewed slices (re-sharded to even parts first, then
        # the library's all-gather: the two-step path), slices whose busiest rank gains nothing from that (direct
        # sends), an empty slice, a remainder past the whole even parts
        cases = {2: [[0, 500, 1000], [0, 100, 1000], [0, 0, 7], [0, 999, 1001]],
                 3: [[0, 333, 666, 999], [0, 50, 120, 1000], [0, 400, 400, 1001], [0, 1, 2, 5]]}[world]
        rng = np.random.default_rng(world)  # ... and twenty seeded random cut sets, the same on every rank
        for _ in range(20):
            total = int(rng.integers(1, 3000))
            inner = np.sort(rng.integers(0, total + 1, world - 1)) if rng.random() < 0.7 else np.sort(rng.choice([0, total], world - 1))
            cases.append([0] + [int(x) for x in inner] + [total])
        took_two_steps = []
        for cc in cases:
            rows_all = torch.arange(cc[-1] * 4, dtype=torch.float32).reshape(cc[-1], 4)
            buf = torch.full_like(rows_all, float("nan"))
            buf[cc[rank]:cc[rank + 1]] = rows_all[cc[rank]:cc[rank + 1]]
            sharded._exchange_row_slices(buf, cc)
            assert torch.equal(buf, rows_all), cc
            took_two_steps.append(cc[-1] // world > 0 and sharded.two_step_pays(cc, cc[-1] // world))
        assert any(took_two_steps) or world == 2
        assert not all(took_two_steps)
        # the replicated operand: every rank brings 1/N of it in, the rest arrives from the other ranks
        B_dev = torch.full_like(B, float("nan"))
        moved = sharded.upload_replicated(B, B_dev)
        assert torch.equal(B_dev, B)
        total = torch.tensor([moved], dtype=torch.int64)
        dist.all_reduce(total)
        assert int(total) == B.numel() * B.element_size()  # the operand crossed the host link once
        nnz = torch.tensor([len(pci)], dtype=torch.int64)
        dist.all_reduce(nnz)
        assert int(nnz) == csr.nnz
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_path_on_gloo_ranks(world, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
