"""Tensor-parallel host logic on CPU: the slice law, the lockstep multi-rank oracle and a
world-size-2 gloo run of the collective wiring (the per-rank linears are the CPU oracle here:
the CUDA kernels cannot run without a GPU)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from scratchy_b200 import synth, tp as tpmod
from scratchy_b200.tp import TpWorld


def test_world_typing():
    # crates/core/tp-world/src/lib.rs:19-95: worlds 1/2/4/8 only, rank inside the world
    for w in (1, 2, 4, 8):
        TpWorld(w, w - 1)
    with pytest.raises(ValueError):
        TpWorld(3, 0)
    with pytest.raises(ValueError):
        TpWorld(4, 4)


def test_slice_law_matches_reference_rows_and_cols():
    # tensor_parallel.rs:1186-1199: Rows = contiguous row block, Cols = per-row column block
    full = torch.arange(8 * 12).reshape(8, 12)
    for w in (2, 4):
        rows = [tpmod.slice_rows(full, TpWorld(w, r)) for r in range(w)]
        cols = [tpmod.slice_cols(full, TpWorld(w, r)) for r in range(w)]
        assert torch.equal(torch.cat(rows, 0), full)
        assert torch.equal(torch.cat(cols, 1), full)
        assert np.array_equal(rows[1].numpy(), oracle.slice_rows(full.numpy(), w, 1))
        assert np.array_equal(cols[1].numpy(), oracle.slice_cols(full.numpy(), w, 1))
    with pytest.raises(ValueError):
        tpmod.slice_rows(torch.zeros(6, 4), TpWorld(4, 0))


def test_affine_row_parallel_requires_whole_groups_per_rank():
    # tensor_parallel.rs:534-537: (K / W) % group == 0
    w = torch.zeros((16, 192 // 8), dtype=torch.int32)
    s = torch.zeros((16, 3), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="group_size"):
        tpmod.shard_affine_row_parallel(w, s, s, TpWorld(2, 0))
    w = torch.zeros((16, 256 // 8), dtype=torch.int32)
    s = torch.zeros((16, 4), dtype=torch.bfloat16)
    a, b, c = tpmod.shard_affine_row_parallel(w, s, s, TpWorld(2, 1))
    assert a.shape == (16, 16) and b.shape == (16, 2) and c.shape == (16, 2)


def lockstep_affine_row_parallel(w, s, b, x, W):
    """Per-rank f32 partials through the oracle, summed in rank order (tensor_parallel.rs:1350-1362)."""
    N, K = w.shape[0], w.shape[1] * 8
    M = x.shape[0]
    parts = []
    for r in range(W):
        wr = oracle.slice_cols(w, W, r)
        sr, br = oracle.slice_cols(s, W, r), oracle.slice_cols(b, W, r)
        xr = oracle.slice_cols(x, W, r)
        _, pf = oracle.affine_qmm_t_b4(wr.view(np.uint8).reshape(-1), sr, br, xr, M, N, K // W, 64, want_f32=True)
        parts.append(pf)
    return oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts)), parts


def lockstep_fp8_row_parallel(wq, ws, x, W):
    N, K = wq.shape
    M = x.shape[0]
    parts = []
    for r in range(W):
        _, pf = oracle.fp8_dynamic_linear(oracle.slice_cols(x, W, r), oracle.slice_cols(wq, W, r), ws, M, N, K // W,
                                          want_f32=True)
        parts.append(pf)
    return oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts)), parts


@pytest.mark.parametrize("W", [2, 4, 8])
def test_ranks_compute_the_unsharded_forward_affine(W):
    """The reference's `two/four/eight_ranks_compute_the_unsharded_forward` (tensor_parallel.rs:1560-1575)
    for this op: column-parallel slices concatenate to the unsharded output exactly; row-parallel
    partials summed in rank order equal it up to f32 re-association."""
    N, K, M = 64, 1024, 3
    w, s, b = synth.affine_int4_weights(N, K, 64, 5)
    x = synth.activations_bf16(M, K, 6)
    full, full_f = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x, M, N, K, 64, want_f32=True)
    cols = []
    for r in range(W):
        wr, sr, br = oracle.slice_rows(w, W, r), oracle.slice_rows(s, W, r), oracle.slice_rows(b, W, r)
        cols.append(oracle.affine_qmm_t_b4(wr.view(np.uint8).reshape(-1), sr, br, x, M, N // W, K, 64))
    assert np.array_equal(np.concatenate(cols, axis=1), full)
    _, parts = lockstep_affine_row_parallel(w, s, b, x, W)
    summed = oracle.allreduce_rank_order(parts)
    assert np.allclose(summed, full_f, rtol=2e-5, atol=1e-4)


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _gloo_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp = TpWorld(world, rank)
        comm = tpmod.TpCommunicator(tp)
        N, K, M = 48, 512, 2
        w, s, b = synth.affine_int4_weights(N, K, 64, 9)
        x = synth.activations_bf16(M, K, 10)
        # shard with the product's slicers (torch), compute the rank's Partial with the oracle
        wt, st, bt = (torch.from_numpy(w.view(np.int32)), torch.from_numpy(s.view(np.int16)),
                      torch.from_numpy(b.view(np.int16)))
        wr, sr, br = tpmod.shard_affine_row_parallel(wt, st, bt, tp)
        xr = tpmod.slice_cols(torch.from_numpy(x.view(np.int16)), tp)
        _, pf = oracle.affine_qmm_t_b4(wr.numpy().view(np.uint8).reshape(-1), sr.numpy().view(np.uint16),
                                       br.numpy().view(np.uint16), xr.numpy().view(np.uint16), M, N, K // world, 64,
                                       want_f32=True)
        part = torch.from_numpy(pf.copy())
        comm.all_reduce(part)
        want, _ = lockstep_affine_row_parallel(w, s, b, x, world)
        got = oracle.f32_to_bf16_bits(part.numpy())
        if world == 2:                      # a + b is the same sum in either order
            ok = bool(np.array_equal(got, want))
        else:                               # the collective's order is not rank order: the 1e-3 bar applies
            gf, wf = oracle.bf16_bits_to_f32(got).astype(np.float64), oracle.bf16_bits_to_f32(want).astype(np.float64)
            ok = bool(np.linalg.norm(gf - wf) / np.linalg.norm(wf) <= 1e-3)
        # AllGather{cols}: the ranks' column blocks in rank order, the padded tail cropped
        rng = np.random.default_rng(5)
        blocks = [rng.integers(0, 65536, size=(3, 10)).astype(np.int32) for _ in range(world)]
        cols = 10 * world - 3
        got = comm.all_gather_cols(torch.from_numpy(blocks[rank]), cols).numpy()
        ok = ok and bool(np.array_equal(got, oracle.allgather_cols_rank_order(blocks, cols)))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_all_gather_law_small_case():
    """tensor_parallel.rs:1363-1386 restated on a case small enough to write out: two ranks, blocks of 3 columns,
    5 real columns: the last block's padded column is cut off, row by row."""
    a = np.array([[1, 2, 3], [7, 8, 9]], np.uint16)
    b = np.array([[4, 5, 99], [10, 11, 99]], np.uint16)
    assert np.array_equal(oracle.allgather_cols_rank_order([a, b], 5), np.array([[1, 2, 3, 4, 5], [7, 8, 9, 10, 11]], np.uint16))
    with pytest.raises(ValueError):
        oracle.allgather_cols_rank_order([a, b], 7)
    comm = tpmod.TpCommunicator(TpWorld(1, 0))
    assert torch.equal(comm.all_gather_cols(torch.from_numpy(a.astype(np.int32)), 2), torch.tensor([[1, 2], [7, 8]], dtype=torch.int32))


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_row_parallel_all_reduce(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(res) == [(r, True) for r in range(world)]


def test_communicator_refuses_world_mismatch():
    with pytest.raises(RuntimeError):
        tpmod.TpCommunicator(TpWorld(2, 0))      # no process group initialised
    tpmod.TpCommunicator(TpWorld(1, 0))          # a single rank needs none
