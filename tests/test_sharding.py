"""Multi-rank logic on CPU: two gloo ranks shard each operation, compute their shard with
the CPU oracle (the GPU kernels are exercised elsewhere), exchange what the design says must
be exchanged, and the assembled result must equal the unsharded one."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mops_b200 import sharding, workloads


def test_batch_range_covers_everything():
    for n, w in [(10, 3), (7, 8), (0, 2), (1 << 22, 8)]:
        parts = [sharding.batch_range(n, w, r) for r in range(w)]
        assert parts[0][0] == 0 and parts[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        sizes = [b - a for a, b in parts]
        assert max(sizes) - min(sizes) <= 1


def test_segment_cuts_keep_rows_whole_and_balance_entries():
    r = np.random.default_rng(0)
    for n_rows, n_entries, world in [(1000, 60000, 8), (5, 100, 4), (50, 10, 3), (3, 1000, 8)]:
        idx = np.sort(r.integers(0, n_rows, n_entries)).astype(np.int32)
        rho, eps = sharding.segment_cuts(idx, n_rows, world)
        assert rho[0] == 0 and rho[-1] == n_rows and eps[0] == 0 and eps[-1] == n_entries
        assert all(a <= b for a, b in zip(rho, rho[1:])) and all(a <= b for a, b in zip(eps, eps[1:]))
        for k in range(world):
            part = idx[eps[k]:eps[k + 1]]
            assert part.size == 0 or (part.min() >= rho[k] and part.max() < rho[k + 1])
        if n_entries >= 100 * world and n_rows >= 10 * world:
            sizes = np.diff(eps)
            assert sizes.max() <= 1.2 * n_entries / world
    with pytest.raises(ValueError):
        sharding.segment_cuts(np.array([3, 1, 2]), 4, 2)


def test_segment_cuts_on_a_large_int32_index_is_a_few_binary_searches():
    """The cut search must not convert the index (NumPy does when the needle has another
    dtype): 2^22 entries, sixteen parts, well under a tenth of a second; the caller that has
    already checked the order can say so; int64 indices give the same cuts."""
    import time
    idx = np.sort(np.random.default_rng(1).integers(0, 1 << 16, 1 << 22)).astype(np.int32)
    t0 = time.perf_counter()
    cuts = sharding.segment_cuts(idx, 1 << 16, 16, known_ascending=True)
    assert time.perf_counter() - t0 < 0.1
    assert cuts == sharding.segment_cuts(idx, 1 << 16, 16)
    assert cuts == sharding.segment_cuts(idx.astype(np.int64), 1 << 16, 16)
    own = sharding.shard_scatter({"A": np.zeros((idx.size, 2)), "i": idx}, "i", 1 << 16, 16, 3, ["A"])[0]
    assert own["A"].flags["OWNDATA"] and own["A"].ctypes.data % 16 == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.mops_oracle import Oracle
    o = Oracle()
    ok = {}

    # SAP: batch sharding, no exchange; gather to compare
    d = workloads.sap(I=257)
    a, b = sharding.batch_range(257, world, rank)
    idx = (d["indices_A"], d["indices_B"], d["indices_output"])
    local = o.sap(d["A"][a:b], d["B"][a:b], d["C"], *idx, 50)
    counts = [sharding.batch_range(257, world, r)[1] - sharding.batch_range(257, world, r)[0]
              for r in range(world)]
    full = sharding.all_gather_rows(torch.from_numpy(local), counts).numpy()
    ok["sap"] = np.array_equal(full, o.sap(d["A"], d["B"], d["C"], *idx, 50))

    # OPSAW: segment sharding; forward gathered; grad_W all-reduced
    d = workloads.opsaw(E=3000, n=40)
    loc, (r0, r1) = sharding.shard_scatter(d, "indices_output", 40, world, rank,
                                           ("A", "B", "indices_W"))
    W_rows = d["W"]  # replicated; the local op writes rows [r0, r1) of the output
    # local forward over the rank's rows: W keeps its global row numbering for indices_W,
    # the output is local -> use a W padded view of the right height for the shape rule
    out_local = o.opsa(loc["A"], loc["B"] * W_rows[loc["indices_W"]], loc["indices_output"], r1 - r0)
    rho, _ = sharding.segment_cuts(d["indices_output"], 40, world)
    full = sharding.all_gather_rows(torch.from_numpy(out_local), np.diff(rho)).numpy()
    want = o.opsaw(d["A"], d["B"], d["W"], d["indices_W"], d["indices_output"])
    ok["opsaw_fwd"] = np.allclose(full, want, rtol=1e-13, atol=1e-13)
    # VJP on the shard: grad_output rows of the rank, full-size partial grad_W
    gO_local = d["grad_output"][r0:r1]
    S = np.einsum("ekl,ek->el", gO_local[loc["indices_output"]], loc["A"])
    gW_partial = np.zeros_like(d["W"])
    np.add.at(gW_partial, loc["indices_W"], S * loc["B"])
    gW = sharding.all_reduce_sum(torch.from_numpy(gW_partial)).numpy()
    _, _, gW_want = o.opsaw_vjp(d["grad_output"], d["A"], d["B"], d["W"], d["indices_W"],
                                d["indices_output"])
    ok["opsaw_gW"] = np.allclose(gW, gW_want, rtol=1e-12, atol=1e-12)

    # SASAW forward: segment sharding with the oracle on the local shard
    d = workloads.sasaw(E=800, n=30, N=60)
    loc, (r0, r1) = sharding.shard_scatter(d, "indices_output_1", 30, world, rank,
                                           ("A", "B", "indices_W_1"))
    # the oracle sizes its output by W.shape[0]: compute on full height, keep the local rows
    shifted = loc["indices_output_1"] + r0
    out = o.sasaw(loc["A"], loc["B"], d["C"], d["W"], d["indices_A"], loc["indices_W_1"],
                  d["indices_W_2"], shifted, d["indices_output_2"], 9)[r0:r1]
    rho, _ = sharding.segment_cuts(d["indices_output_1"], 30, world)
    full = sharding.all_gather_rows(torch.from_numpy(np.ascontiguousarray(out)), np.diff(rho)).numpy()
    want = o.sasaw(d["A"], d["B"], d["C"], d["W"], d["indices_A"], d["indices_W_1"],
                   d["indices_W_2"], d["indices_output_1"], d["indices_output_2"], 9)
    ok["sasaw_fwd"] = np.allclose(full, want, rtol=1e-13, atol=1e-13)

    if rank == 0:
        results.update(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded_results():
    world = 2
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        got = dict(results)
    assert got and all(got.values()), got


# ------------------------------------------------------------------ shards on a GPU
SHARD_CASES = {"hpe": dict(I=9000, N=30, J=200, K=4), "sap": dict(I=9000),
               "opsa": dict(J=200000, nO=3000), "opsaw": dict(E=120000, n=2000),
               "sasaw": dict(E=60000, n=1000)}


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("op", sorted(SHARD_CASES))
def test_shards_run_on_the_gpu_assemble_to_the_unsharded_result(oracle, op, world):
    """The ranks' shards of one problem (cut by mops_b200.sharding exactly as bench.py's
    strong-scaling leg cuts them) are run one after the other on one GPU; the assembled
    output, the concatenated per-row / per-entry gradients and the summed grad_W must equal
    the unsharded GPU result, and match the oracle on sub-ranges."""
    import subrange
    from conftest import assert_parity
    from helpers import run_library, to_dev
    d = workloads.GENERATORS[op](**SHARD_CASES[op])
    full = run_library(op, to_dev(d, np.float64))
    parts = []
    for rank in range(world):
        if op in ("hpe", "sap"):
            a, b = sharding.batch_range(d["A"].shape[0], world, rank)
            loc = {k: (v[a:b] if k in ("A", "B", "grad_output") else v) for k, v in d.items()}
        else:
            key = "indices_output_1" if op == "sasaw" else "indices_output"
            n_rows = d["output_size"] if op == "opsa" else d["W"].shape[0]
            loc, (r0, r1) = sharding.shard_scatter(d, key, n_rows, world, rank,
                                                   ("A", "B", "indices_W", "indices_W_1"))
            if op == "opsa":   # the output itself is sharded by rows
                loc["output_size"] = r1 - r0
                loc["grad_output"] = d["grad_output"][r0:r1]
            else:              # W couples all rows: full-height output, other rows stay zero
                loc[key] = loc[key] + r0
        parts.append(run_library(op, to_dev(loc, np.float64)))
    cat = lambda k: np.concatenate([p[k] for p in parts], axis=0)
    got = {}
    if op in ("hpe", "sap", "opsa"):
        got = {k: cat(k) for k in full}
    else:
        got["output"] = sum(p["output"] for p in parts)
        got["grad_A"], got["grad_B"] = cat("grad_A"), cat("grad_B")
        got["grad_W"] = sum(p["grad_W"] for p in parts)
    for k in full:
        assert_parity(got[k], full[k], f"{op}/{k} from {world} shards")
    subrange.check_case(oracle, op, d, got)
