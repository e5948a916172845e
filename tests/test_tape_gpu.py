"""GPU parity of the one-launch matvec tape (`scr_linear_affine_b4_tape`) against the CPU oracle.

Every job's output is checked against the oracle applied to the bits the job actually read (its x
buffer after the run), so a chain does not compound tolerances; outputs are pre-filled with NaN, so a
job that started before its producer had stored would show.  Bar: relative L2 1e-3 per job (bf16
outputs of an f32-accumulated sum), bit-identical across replays.
"""
import numpy as np
import pytest

import oracle
from scratchy_b200 import synth
from util import bf16_dev, bits_of, rel_l2, u32_dev

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3
NAN_BITS = 0x7FC0


def _linear(N, K, seed):
    from scratchy_b200 import AffineQuantLinear
    w, s, b = synth.affine_int4_weights(N, K, 64, seed)
    return AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4), (w, s, b)


def _decoder_like_tape(M, hidden, q_dim, kv_dim, inter, n_layers, seed):
    """q, k, v <- x; o <- q (after q, k, v); gate, up <- o; down <- gate (after gate, up); next layer <- down."""
    import torch
    jobs, host = [], []
    x0 = bf16_dev(synth.activations_bf16(M, hidden, seed))
    x_in, x_dep = x0, []
    for layer in range(n_layers):
        base = len(jobs)
        shapes = [(q_dim, hidden), (kv_dim, hidden), (kv_dim, hidden), (hidden, q_dim), (inter, hidden), (inter, hidden),
                  (hidden, inter)]
        ys = [torch.empty((M, n), dtype=torch.bfloat16, device="cuda") for n, _ in shapes]
        xs = [x_in, x_in, x_in, ys[0], ys[3], ys[3], ys[4]]
        deps = [x_dep, x_dep, x_dep, [base, base + 1, base + 2], [base + 3], [base + 3], [base + 4, base + 5]]
        for i, (n, k) in enumerate(shapes):
            lin, raw = _linear(n, k, synth.seed_for("tape", seed, layer, i))
            jobs.append((lin, xs[i], ys[i], deps[i]))
            host.append((raw, n, k))
        x_in, x_dep = ys[6], [base + 6]
    return jobs, host


def _check_jobs(jobs, host, M):
    for j, ((lin, x, y, _), ((w, s, b), n, k)) in enumerate(zip(jobs, host)):
        xb = bits_of(x)[:M]
        assert not np.any((xb & 0x7FFF) > 0x7F80), f"job {j} read an input that was never written"
        want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, xb, M, n, k, 64)
        err = rel_l2(bits_of(y)[:M], want)
        assert err <= REL_L2_TOL, f"job {j} ({n}x{k}): rel-L2 {err:.3e}"


@pytest.mark.parametrize("M,max_rows,hidden,q_dim,kv_dim,inter,n_layers", [
    (1, 1, 256, 256, 64, 1088, 2),          # few row-blocks per job; K = 1088 ends in a partial ring stage
    (5, 8, 256, 384, 128, 512, 3),          # fewer rows than the buffers hold
    (8, 8, 512, 512, 72, 8192, 1),          # 8192 rows: more row-blocks than CTAs; 72 rows: a ragged last row-block
    (11, 16, 256, 256, 64, 512, 2),         # the two-tile (up to 16 rows) variant
    (16, 16, 192, 320, 64, 640, 2),
])
def test_decoder_like_chain(M, max_rows, hidden, q_dim, kv_dim, inter, n_layers):
    import torch
    from scratchy_b200 import AffineTape, _lib
    jobs, host = _decoder_like_tape(max_rows, hidden, q_dim, kv_dim, inter, n_layers, seed=M * 100 + hidden)
    tape = AffineTape(jobs, max_rows=max_rows)
    runs = []
    for _ in range(3):                       # replays: the kernel leaves its counters cleared
        for _, _, y, _ in jobs:
            y.view(torch.int16).fill_(NAN_BITS)
        tape.run(M)
        torch.cuda.synchronize()
        _lib.context(0).device_status(None)
        runs.append([bits_of(y)[:M].copy() for _, _, y, _ in jobs])
    _check_jobs(jobs, host, M)
    for other in runs[1:]:
        assert all(np.array_equal(a, b) for a, b in zip(runs[0], other)), "replays must give the same bits"
    tape.close()


def test_tape_replayed_from_a_cuda_graph_llama_layer_shapes():
    """Two Llama-3.2-3B layers (the headline workload's shapes) as one tape, captured and replayed."""
    import torch
    from scratchy_b200 import AffineTape, _lib
    jobs, host = _decoder_like_tape(1, 3072, 3072, 1024, 8192, 2, seed=7)
    tape = AffineTape(jobs, max_rows=1)
    tape.run()
    torch.cuda.synchronize()
    first = [bits_of(y).copy() for _, _, y, _ in jobs]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        tape.run()
    for _ in range(3):
        for _, _, y, _ in jobs:
            y.view(torch.int16).fill_(NAN_BITS)
        graph.replay()
    torch.cuda.synchronize()
    _lib.context(0).device_status(None)
    assert all(np.array_equal(a, bits_of(y)) for a, (_, _, y, _) in zip(first, jobs))
    _check_jobs(jobs, host, 1)
    # against the one-launch-per-linear path on the same inputs: the same values up to the summation order
    for lin, x, y, _ in jobs[:7]:
        sep = lin.forward(x)
        torch.cuda.synchronize()
        assert rel_l2(bits_of(y), bits_of(sep)) <= REL_L2_TOL
    tape.close()


def test_tape_arguments_are_checked():
    import torch
    from scratchy_b200 import AffineTape, _lib
    lin, _ = _linear(64, 128, 1)
    x = torch.zeros((2, 128), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.ScratchyCudaError) as e:
        AffineTape([(lin, x, y, [0])], max_rows=2)               # a job cannot wait for itself
    assert e.value.status == -1
    x17 = torch.zeros((17, 128), dtype=torch.bfloat16, device="cuda")
    y17 = torch.zeros((17, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.ScratchyCudaError) as e:
        AffineTape([(lin, x17, y17, [])], max_rows=17)           # beyond the matvec path
    assert e.value.status == -7
    tape = AffineTape([(lin, x, y, [])], max_rows=2)
    with pytest.raises(_lib.ScratchyCudaError) as e:
        tape.run(3)
    assert e.value.status == -2
    with pytest.raises(ValueError):
        AffineTape([(lin, x, y[:, :32], [])], max_rows=2)
    tape.close()
