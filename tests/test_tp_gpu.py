"""Tensor-parallel parity on the GPU.

One-GPU part: the `Partial` (f32) outputs of a row-parallel slice, summed in rank order on the
host, must match the lockstep oracle at the same world size (parity is per world size: each
rank quantises its own K-slice per token, so fp8 results differ slightly from TP=1 by design).
Multi-GPU part (needs >= 2 devices, skipped otherwise): two processes, NCCL all-reduce.
"""
import os
import socket

import numpy as np
import pytest

import oracle
from scratchy_b200 import synth
from test_tp_cpu import lockstep_affine_row_parallel, lockstep_fp8_row_parallel
from util import bf16_dev, bits_of, rel_l2, to_dev, u32_dev

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


@pytest.mark.parametrize("W,M", [(2, 1), (8, 4), (4, 40)])
def test_affine_row_parallel_partials_one_gpu(W, M):
    import torch
    from scratchy_b200 import AffineQuantLinear
    N, K = 256, 2048
    w, s, b = synth.affine_int4_weights(N, K, 64, 31)
    x = synth.activations_bf16(M, K, 32)
    parts = []
    for r in range(W):
        lin = AffineQuantLinear.from_tensors(u32_dev(oracle.slice_cols(w, W, r)), bf16_dev(oracle.slice_cols(s, W, r)),
                                             bf16_dev(oracle.slice_cols(b, W, r)))
        parts.append(lin.forward_partial(bf16_dev(oracle.slice_cols(x, W, r)).reshape(M, K // W)).cpu().numpy())
    torch.cuda.synchronize()
    got = oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts))
    want, _ = lockstep_affine_row_parallel(w, s, b, x, W)
    assert rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("W,M", [(2, 1), (8, 16), (4, 40)])
def test_fp8_row_parallel_partials_one_gpu(W, M):
    import torch
    from scratchy_b200 import Fp8Linear
    N, K = 256, 2048
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, 33))
    x = synth.activations_bf16(M, K, 34)
    parts = []
    for r in range(W):
        lin = Fp8Linear.from_tensors(to_dev(oracle.slice_cols(wq, W, r)), to_dev(ws))
        parts.append(lin.forward_partial(bf16_dev(oracle.slice_cols(x, W, r)).reshape(M, K // W)).cpu().numpy())
    torch.cuda.synchronize()
    got = oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts))
    want, _ = lockstep_fp8_row_parallel(wq, ws, x, W)
    assert rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("name,M", [("o", 1), ("o", 4), ("o", 32), ("down", 1), ("down", 4)])
def test_llama_70b_row_parallel_shards_at_tp8(name, M):
    """The Llama-3-70B row-parallel shapes of the tensor-parallel benchmark configuration at world size 8 (o: 1024 of
    8192 input features per rank, down: 3584 of 28672; 8192 outputs), every rank's shard run on this one GPU:
    (i) the f32 partials summed in rank order and rounded once against the lockstep oracle, (ii) every rank's partial
    against the oracle's, (iii) for the self-quantising matvec sizes, the matvec with the exchange in its epilogue on
    a one-rank communicator against the ORACLE's rounded partial of that rank (not against the partial path)."""
    import torch
    from scratchy_b200 import Fp8Linear, tp as tpmod
    W = 8
    K, N = synth.LLAMA_3_70B[name]
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, synth.seed_for("tp70", N, K)))
    x = synth.activations_bf16(M, K, synth.seed_for("tp70x", N, K, M))
    want, want_parts = lockstep_fp8_row_parallel(wq, ws, x, W)
    dev = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=M * N)
    parts = []
    for r in range(W):
        lin = Fp8Linear.from_tensors(to_dev(oracle.slice_cols(wq, W, r)), to_dev(ws))
        xr = bf16_dev(oracle.slice_cols(x, W, r)).reshape(M, K // W)
        part = lin.forward_partial(xr)
        parts.append(part.cpu().numpy())
        assert rel_l2(oracle.f32_to_bf16_bits(parts[-1]), oracle.f32_to_bf16_bits(want_parts[r])) <= REL_L2_TOL, f"rank {r} partial"
        if one.fp8_linear_all_reduce_supported(lin, M):
            fused = one.fp8_linear_all_reduce(lin, xr)
            torch.cuda.synchronize()
            assert rel_l2(bits_of(fused), oracle.f32_to_bf16_bits(want_parts[r])) <= REL_L2_TOL, f"rank {r} fused"
    torch.cuda.synchronize()
    got = oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts))
    r = rel_l2(got, want)
    print(f"70B {name} TP=8 M={M} rel_l2={r:.3e}")
    assert r <= REL_L2_TOL
    __import__("scratchy_b200")._lib.context(0).device_status(None)
    one.close()


def _nccl_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    from scratchy_b200 import AffineQuantLinear, Fp8Linear, tp as tpmod
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")           # a rank that fails must not die bound to a multicast object
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        tp = tpmod.TpWorld(world, rank)
        comm = tpmod.TpCommunicator(tp)
        N, K, M = 512, 4096, 8
        ok = True
        w, s, b = synth.affine_int4_weights(N, K, 64, 41)
        x = synth.activations_bf16(M, K, 42)
        dev = torch.device("cuda", rank)
        wt = torch.from_numpy(w.view(np.int32)).to(dev)
        st = torch.from_numpy(s.view(np.int16)).view(torch.bfloat16).to(dev)
        bt = torch.from_numpy(b.view(np.int16)).view(torch.bfloat16).to(dev)
        xt = torch.from_numpy(x.view(np.int16)).view(torch.bfloat16).to(dev)
        lin = AffineQuantLinear.from_tensors(*tpmod.shard_affine_row_parallel(wt, st, bt, tp))
        y = tpmod.RowParallel(lin, comm).forward(tpmod.slice_cols(xt, tp))
        want, _ = lockstep_affine_row_parallel(w, s, b, x, world)
        ok &= rel_l2(y.view(torch.int16).cpu().numpy().view(np.uint16), want) <= REL_L2_TOL
        wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, 43))
        flin = Fp8Linear.from_tensors(*tpmod.shard_fp8_row_parallel(torch.from_numpy(wq).to(dev),
                                                                    torch.from_numpy(ws).to(dev), tp))
        y = tpmod.RowParallel(flin, comm).forward(tpmod.slice_cols(xt, tp))
        want, _ = lockstep_fp8_row_parallel(wq, ws, x, world)
        ok &= rel_l2(y.view(torch.int16).cpu().numpy().view(np.uint16), want) <= REL_L2_TOL
        # the one-shot exchange over peer memory: rank-ordered sum, bit for bit, eagerly and replayed from a graph
        one = tpmod.OneShotAllReduce(tp, dev, max_elems=40 * 1024)
        rng = np.random.default_rng(7)
        parts = [rng.standard_normal((5, 1024)).astype(np.float32) * (1.0 + r) for r in range(world)]
        want_bits = oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts))
        mine = torch.from_numpy(parts[rank]).to(dev)
        for _ in range(3):                                   # consecutive calls alternate the receive halves
            got = one.all_reduce(mine)
            ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want_bits))
        # a payload beyond the packet form (dense stores + one flag per CTA and rank), interleaved with the small one
        big = [rng.standard_normal((40, 1024)).astype(np.float32) * (1.0 + r) for r in range(world)]
        big_bits = oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(big))
        big_mine = torch.from_numpy(big[rank]).to(dev)
        for _ in range(3):
            got = one.all_reduce(big_mine)
            ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), big_bits))
            got = one.all_reduce(mine)
            ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want_bits))
        # the other collective, AllGather{cols}: column blocks side by side in rank order, the padded tail cropped;
        # 16-byte rows, odd rows (the scalar form), and an N-split vocabulary head through ColumnParallel
        for rows_g, lc_g, cols_g in [(3, 1024, world * 1024), (5, 64, world * 64 - 24), (2, 37, world * 37 - 5)]:
            blocks = [synth.f32_to_bf16_bits(rng.standard_normal((rows_g, lc_g)).astype(np.float32) + r) for r in range(world)]
            want_g = oracle.allgather_cols_rank_order(blocks, cols_g)
            mine_g = torch.from_numpy(blocks[rank].view(np.int16)).view(torch.bfloat16).to(dev)
            for _ in range(2):
                got = one.all_gather_cols(mine_g, cols_g)
                ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want_g))
                got = one.all_reduce(mine)                   # interleaved with the all-reduce on the same communicator
                ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want_bits))
            got = comm.all_gather_cols(mine_g, cols_g)       # the process group's form gives the same bytes
            ok &= bool(np.array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want_g))
        vocab = 64 * world
        wv, sv, bv = synth.affine_int4_weights(vocab, K, 64, 47)
        head = AffineQuantLinear.from_tensors(*tpmod.shard_affine_column_parallel(
            torch.from_numpy(wv.view(np.int32)).to(dev), torch.from_numpy(sv.view(np.int16)).view(torch.bfloat16).to(dev),
            torch.from_numpy(bv.view(np.int16)).view(torch.bfloat16).to(dev), tp))
        logits = tpmod.ColumnParallel(head, comm, one_shot=one, gather_cols=vocab).forward(xt)
        want_logits = oracle.affine_qmm_t_b4(wv.view(np.uint8).reshape(-1), sv, bv, x, M, vocab, K, 64)
        ok &= rel_l2(logits.view(torch.int16).cpu().numpy().view(np.uint16), want_logits) <= REL_L2_TOL
        got16 = torch.empty((5, 1024), dtype=torch.bfloat16, device=dev)
        got32 = torch.empty((5, 1024), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            one.all_reduce(mine, out_bf16=got16, out_f32=got32)
        for _ in range(4):
            got16.zero_()
            graph.replay()
            torch.cuda.synchronize()
            ok &= bool(np.array_equal(got16.view(torch.int16).cpu().numpy().view(np.uint16), want_bits))
            ok &= bool(np.array_equal(got32.cpu().numpy(), oracle.allreduce_rank_order(parts)))
        y = tpmod.RowParallel(flin, comm, one_shot=one).forward(tpmod.slice_cols(xt, tp))
        ok &= rel_l2(y.view(torch.int16).cpu().numpy().view(np.uint16), want) <= REL_L2_TOL
        # matvec + exchange in one launch: the bits of the partial matvec followed by the one-shot exchange,
        # for a persistent grid (N = 8192: more row-blocks than CTAs) and a cluster-split one (N = 512),
        # interleaved with stand-alone exchanges on the same communicator, eagerly and from a graph
        for n_out, m_rows in [(512, 3), (8192, 1), (8192, 2)]:
            wq2, ws2 = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(n_out, K, 50 + m_rows))
            f2 = Fp8Linear.from_tensors(*tpmod.shard_fp8_row_parallel(torch.from_numpy(wq2).to(dev),
                                                                      torch.from_numpy(ws2).to(dev), tp))
            xl = tpmod.slice_cols(xt[:m_rows], tp).contiguous()
            ref = one.all_reduce(f2.forward_partial(xl))
            ok &= one.fp8_linear_all_reduce_supported(f2, m_rows)
            for _ in range(3):
                got = one.fp8_linear_all_reduce(f2, xl)
                ok &= bool(torch.equal(got.view(torch.int16), ref.view(torch.int16)))
            fused_out = torch.empty_like(ref)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                one.fp8_linear_all_reduce(f2, xl, out=fused_out)
                one.all_reduce(mine, out_bf16=got16)
            for _ in range(3):
                fused_out.zero_()
                graph.replay()
                torch.cuda.synchronize()
                ok &= bool(torch.equal(fused_out.view(torch.int16), ref.view(torch.int16)))
                ok &= bool(np.array_equal(got16.view(torch.int16).cpu().numpy().view(np.uint16), want_bits))
            want2, _ = lockstep_fp8_row_parallel(wq2, ws2, x[:m_rows], world)
            ok &= rel_l2(fused_out.view(torch.int16).cpu().numpy().view(np.uint16), want2) <= REL_L2_TOL
        torch.cuda.synchronize()
        _lib_ctx = __import__("scratchy_b200")._lib.context(rank)
        _lib_ctx.device_status(None)                         # no bounded flag wait ran out
        one.close()
        q.put((rank, bool(ok)))
    except BaseException as exc:                             # a rank that raises reports it at once: the parent must not wait
        import traceback
        q.put((rank, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))
        q.close()
        q.join_thread()
        torch.cuda.synchronize()                             # leave with none of this rank's kernels in flight
        os._exit(1)                                          # no collective teardown with a peer that may be mid-call
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_nccl_row_parallel(world):
    """One process per GPU at world sizes 2, 4 and 8 (each needs that many devices): both exchange paths and the
    matvec with the exchange in its epilogue against the lockstep oracle at the same world size."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    for _ in procs:
        res.append(q.get(timeout=240))
        if res[-1][1] is not True:                           # one rank failed: the others may be waiting for it
            break
    for p in procs:
        p.join(timeout=20 if len(res) == len(procs) and all(r[1] is True for r in res) else 1)
        if p.is_alive():
            p.kill()                                         # exactly the processes this test started
    assert sorted(res) == [(r, True) for r in range(world)], res


def test_ranks_as_threads_of_one_process_connect_locally():
    """The reference's executor drives its ranks as threads of ONE process (crates/serving/worker/src/threadpool.rs:1-16):
    such ranks cannot open each other's IPC handles and connect through raw device pointers instead
    (`scr_tp_comm_connect_local`).  World 1 on one GPU always; two host threads on two GPUs when they exist."""
    import threading
    import torch
    from scratchy_b200 import _lib, tp as tpmod
    dev0 = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev0, max_elems=8192, connect=False)
    one.connect_local([one.base], [0])
    part = torch.from_numpy(np.random.default_rng(1).standard_normal((2, 1024)).astype(np.float32)).to(dev0)
    got = one.all_reduce(part)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(got), oracle.f32_to_bf16_bits(part.cpu().numpy()))
    one.close()
    if torch.cuda.device_count() < 2:
        return
    world = 2
    rng = np.random.default_rng(11)
    small = [rng.standard_normal((3, 1024)).astype(np.float32) * (1.0 + r) for r in range(world)]
    large = [rng.standard_normal((40, 1024)).astype(np.float32) * (1.0 + r) for r in range(world)]
    blocks = [synth.f32_to_bf16_bits(rng.standard_normal((4, 264)).astype(np.float32)) for _ in range(world)]
    comms, results, gathered, errors = [None] * world, [None] * world, [None] * world, []
    gate = threading.Barrier(world)

    def rank_thread(r):
        try:
            dev = torch.device("cuda", r)
            torch.cuda.set_device(dev)
            comms[r] = tpmod.OneShotAllReduce(tpmod.TpWorld(world, r), dev, max_elems=64 * 1024, connect=False)
            gate.wait()
            comms[r].connect_local([c.base for c in comms], list(range(world)))
            gate.wait()
            out = []
            for parts in (small, large, small):                 # packets, dense stores + flags, packets again
                got = comms[r].all_reduce(torch.from_numpy(parts[r]).to(dev))
                torch.cuda.synchronize(dev)
                out.append(bits_of(got))
            gathered[r] = bits_of(comms[r].all_gather_cols(bf16_dev(blocks[r]).to(dev), 2 * 264 - 8))
            torch.cuda.synchronize(dev)
            results[r] = out
            _lib.context(r).device_status(None)
            gate.wait()                                          # nobody frees a buffer a peer may still write
            comms[r].close()
        except Exception as exc:                                 # a failing rank must not leave the other at the barrier
            errors.append(exc)
            gate.abort()

    threads = [threading.Thread(target=rank_thread, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    for r in range(world):
        for got, parts in zip(results[r], (small, large, small)):
            assert np.array_equal(got, oracle.f32_to_bf16_bits(oracle.allreduce_rank_order(parts)))
        assert np.array_equal(gathered[r], oracle.allgather_cols_rank_order(blocks, 2 * 264 - 8))


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_call_works():
    """Failure detection without a fault: a world-2 communicator on ONE GPU whose second "peer" is the rank's own
    buffer, so nothing ever writes rank 1's slots.  With a short poll limit the exchange kernels give up, return,
    and `scr_device_status` reports SCR_E_TIMEOUT; the context stays usable and the next call on an ordinary
    communicator gives the right bits."""
    import torch
    from scratchy_b200 import Fp8Linear, _lib, tp as tpmod
    dev = torch.device("cuda", 0)
    ctx = _lib.context(0)
    ctx.device_status(None)
    lame = tpmod.OneShotAllReduce(tpmod.TpWorld(2, 0), dev, max_elems=64 * 1024, connect=False)
    lame.connect_local([lame.base, lame.base], [0, 0])
    lame.set_wait_limit(1 << 12)
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(512, 1024, 9))
    lin = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws))
    x = bf16_dev(synth.activations_bf16(1, 1024, 10)).reshape(1, 1024)
    calls = [lambda: lame.all_reduce(torch.ones((2, 1024), device=dev)),           # packets
             lambda: lame.all_reduce(torch.ones((40, 1024), device=dev)),          # dense stores + flags
             lambda: lame.fp8_linear_all_reduce(lin, x)]                           # the matvec that exchanges in its epilogue
    for i, call in enumerate(calls):
        call()
        with pytest.raises(_lib.ScratchyCudaError) as e:
            lame.check_health()
        assert e.value.status == -8, f"call {i}: expected SCR_E_TIMEOUT, got {e.value.name}"
        ctx.device_status(None)                                                    # read and cleared: healthy again
    lame.close()
    good = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=8192)
    part = torch.from_numpy(np.random.default_rng(2).standard_normal((4, 1024)).astype(np.float32)).to(dev)
    got = good.all_reduce(part)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(got), oracle.f32_to_bf16_bits(part.cpu().numpy()))
    ctx.device_status(None)
    good.close()


@pytest.mark.parametrize("rows,lc,cols", [(1, 128256, 128256), (4, 4096, 4000), (3, 37, 30), (16, 8, 8)])
def test_all_gather_cols_single_rank(rows, lc, cols):
    """`SubOp::AllGather{cols}` at world 1 is the crop of the padded block; the oracle's law gives the bytes."""
    import torch
    from scratchy_b200 import _lib, tp as tpmod
    dev = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=256 * 1024)
    blk = synth.f32_to_bf16_bits(np.random.default_rng(rows * lc).standard_normal((rows, lc)).astype(np.float32))
    for _ in range(2):
        got = one.all_gather_cols(bf16_dev(blk), cols)
        torch.cuda.synchronize()
        assert np.array_equal(bits_of(got), oracle.allgather_cols_rank_order([blk], cols))
    with pytest.raises(_lib.ScratchyCudaError) as e:
        one.all_gather_cols(bf16_dev(blk), lc + 1)               # one block of lc columns cannot restore lc + 1
    assert e.value.name == "SCR_E_SHAPE"
    one.close()


def test_one_shot_all_reduce_single_rank():
    """World size 1 runs the whole kernel on one GPU (push to itself, flag, wait, sum of one operand):
    indexing, the device-side call counter, the two receive halves and graph replay."""
    import torch
    from scratchy_b200 import _lib, tp as tpmod
    dev = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=300 * 1024)
    rng = np.random.default_rng(3)
    for shape in [(1, 8192), (16, 8192), (3, 1028), (1, 4), (37, 8192)]:      # 37 x 8192 > 256 CTAs x 1024: strided slices
        part = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dev)
        got = one.all_reduce(part)
        f32 = torch.empty(shape, dtype=torch.float32, device=dev)
        one.all_reduce(part, out_f32=f32)
        torch.cuda.synchronize()
        assert np.array_equal(bits_of(got), oracle.f32_to_bf16_bits(part.cpu().numpy()))
        assert torch.equal(f32, part)
    part = torch.from_numpy(rng.standard_normal((2, 8192)).astype(np.float32)).to(dev)
    out = torch.empty((2, 8192), dtype=torch.bfloat16, device=dev)
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        one.all_reduce(part, out_bf16=out)
    for i in range(5):
        part.copy_(torch.from_numpy(rng.standard_normal((2, 8192)).astype(np.float32)))
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(bits_of(out), oracle.f32_to_bf16_bits(part.cpu().numpy())), f"replay {i}"
    _lib.context(0).device_status(None)
    with pytest.raises(_lib.ScratchyCudaError):
        one.all_reduce(torch.zeros(301 * 1024, device=dev))                    # beyond max_elems
    with pytest.raises(_lib.ScratchyCudaError):
        one.all_reduce(torch.zeros(6, device=dev))                             # not a multiple of 4
    one.close()


@pytest.mark.parametrize("N,K,M", [(8192, 1024, 1), (8192, 3584, 4), (512, 4096, 3), (72, 1024, 2), (8192, 14336, 1)])
def test_fp8_matvec_with_exchange_single_rank(N, K, M):
    """World size 1 runs the whole fused kernel on one GPU (push to itself, flag, wait, sum of one operand):
    the result is the rounded partial, bit for bit, for persistent and cluster-split grids, eagerly,
    interleaved with stand-alone exchanges, and replayed from a CUDA graph."""
    import torch
    from scratchy_b200 import Fp8Linear, _lib, tp as tpmod
    dev = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=4 * 8192)
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, N + K))
    lin = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws))
    x = bf16_dev(synth.activations_bf16(M, K, 5)).reshape(M, K)
    want = tpmod.partial_to_bf16(lin.forward_partial(x))
    assert one.fp8_linear_all_reduce_supported(lin, M)
    for i in range(3):
        got = one.fp8_linear_all_reduce(lin, x)
        if i == 1:
            one.all_reduce(torch.zeros(8, device=dev))            # a stand-alone call in between: the halves keep alternating
        torch.cuda.synchronize()
        assert np.array_equal(bits_of(got), bits_of(want)), f"call {i}"
    out = torch.zeros_like(want)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        one.fp8_linear_all_reduce(lin, x, out=out)
    for i in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(bits_of(out), bits_of(want)), f"replay {i}"
    _lib.context(0).device_status(None)
    one.close()


def test_fp8_matvec_with_exchange_refuses_what_it_cannot_fuse():
    import torch
    from scratchy_b200 import Fp8Linear, _lib, tp as tpmod
    dev = torch.device("cuda", 0)
    one = tpmod.OneShotAllReduce(tpmod.TpWorld(1, 0), dev, max_elems=8192)
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(256, 1024, 1))
    lin = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws))
    with pytest.raises(_lib.ScratchyCudaError) as e:
        one.fp8_linear_all_reduce(lin, torch.zeros((8, 1024), dtype=torch.bfloat16, device=dev))     # 8 rows: not self-quantising
    assert e.value.status == -7
    big = Fp8Linear.from_tensors(to_dev(np.repeat(wq, 64, axis=0)), to_dev(np.repeat(ws, 64)))       # 16384 outputs > max_elems
    with pytest.raises(_lib.ScratchyCudaError) as e:
        one.fp8_linear_all_reduce(big, torch.zeros((1, 1024), dtype=torch.bfloat16, device=dev))
    assert e.value.status == -2
    assert not one.fp8_linear_all_reduce_supported(lin, 8)
    one.close()
