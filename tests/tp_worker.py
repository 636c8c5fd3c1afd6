"""Worker of tests/test_tp.py (one process per rank, launched by torch.distributed.run).

mode "cpu": gloo only -- the rendezvous helpers and the row-parallel rule on the oracle: every rank quantises its
K-slice, the float partial sums are all-reduced over gloo and must equal the oracle's tp-way split.
mode "gpu": the tensor-parallel decoder on one GPU per rank over NCCL against the oracle's tp-way split.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from nn_b200 import dist  # noqa: E402
from nn_b200.gpt import GptConfig  # noqa: E402
from oracle import model as om, oracle as orc  # noqa: E402


def cpu_mode():
    import torch
    import torch.distributed as td
    rank, world, _ = dist.env_rank()
    payload = bytes(range(128)) if rank == 0 else None
    assert dist.broadcast_bytes(payload, 128) == bytes(range(128))
    assert dist.all_reduce_max(float(rank)) == float(world - 1)
    # row-parallel Linear: this rank's shard, partial sums reduced over gloo
    M, K, N = 5, 256, 48
    x = orc.round_bf16(orc.normal((M, K), 1))
    w = orc.normal((K, N), 2, 0.02)
    bias = orc.normal((N,), 3, 0.01)
    ks = K // world
    xq, xs = orc.quantize_rows_i8(np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks]))
    wq, ws = orc.quantize_rows_i8(np.ascontiguousarray(w[rank * ks:(rank + 1) * ks].T))
    part = torch.from_numpy(orc.dequant_epilogue(orc.qmatmul_i8_acc(xq, wq), xs, ws))
    td.all_reduce(part)
    got = part.numpy() + bias[None, :]
    exp = om._q_linear(x, w, bias, tp=world, split="row")
    assert orc.close(exp, got, 1e-5), orc.max_err(exp, got)
    dist.barrier()
    print(f"rank {rank}: cpu ok")


def gpu_mode():
    from nn_b200.device import Device
    from nn_b200.gpt import GptW8A8
    rank, world, local = dist.env_rank()
    dev = Device(local)
    comm, rank, world = dist.init_comm(dev)
    cfg = GptConfig(vocab=320, dim=512, heads=4, layers=2, ff_dim=1024, context=32)
    w = om.make_weights(cfg, seed=4)
    B = 3
    prompt = orc.token_ids((B, 12), 44, cfg.vocab).astype(np.int64)
    ref = om.W8A8Decoder(cfg, w, B, tp=world)
    exp, exp_resets = ref.generate(prompt, 30)
    m = GptW8A8(dev, cfg, w, B, max_prefill=16, tp_rank=rank, tp_size=world, comm=comm)
    m.prefill(prompt.astype(np.int32))
    dev.synchronize()
    local_logits = m.read_logits()
    full = ref.logit_trace[0][:, rank * m.v_loc:(rank + 1) * m.v_loc]
    assert orc.close(full, local_logits, 5e-2), orc.max_err(full, local_logits)
    got, resets = m.generate(prompt, 30, use_graph=True)
    assert resets == exp_resets == 1
    # every rank must hold the same tokens (the merge is deterministic); agreement with the oracle is exact unless a
    # near-tie flipped, which the logits check above bounds
    import torch
    import torch.distributed as td
    mine = torch.from_numpy(got.astype(np.int64))
    ref0 = mine.clone()
    td.broadcast(ref0, 0)
    assert torch.equal(mine, ref0)
    # Greedy tokens equal the oracle's up to the first step where the oracle's two best logits are closer than the
    # logit tolerance (a near-tie may flip, and the sequences differ from there on): check every sequence up to that
    # step and that the step really is a near-tie.
    agree = float((got == exp).mean())
    for b in range(B):
        diff = np.nonzero(got[b] != exp[b])[0]
        if diff.size:
            s = int(diff[0])
            top2 = np.sort(ref.logit_trace[s][b])[-2:]
            assert top2[1] - top2[0] <= 2 * 5e-2 * max(1.0, abs(float(top2[1]))), \
                f"sequence {b} leaves the oracle's tokens at step {s} without a near-tie (gap {top2[1] - top2[0]:.3g})"
    assert m.peer is not None, "few-row passes must have used the peer-memory exchange"
    m.close()
    # the same model over NCCL inside the layers (all-reduce, bias + residual, LayerNorm as three kernels) is held to the
    # oracle in the same way (the peer-memory kernel adds the ranks' rows in rank order, NCCL in its own)
    m2 = GptW8A8(dev, cfg, w, B, max_prefill=16, tp_rank=rank, tp_size=world, comm=comm, peer_exchange=False)
    assert m2.peer is None
    m2.prefill(prompt.astype(np.int32))
    dev.synchronize()
    assert orc.close(full, m2.read_logits(), 5e-2), orc.max_err(full, m2.read_logits())
    m2.close()
    # ---- prompt read by batch sharding, keys / values delivered into the head-sharded caches over peer memory: the pages
    # this rank ends up with must equal, bit for bit, the pages of its heads in a ONE-GPU model's cache (which is what
    # every rank computed for its share of the sequences), the first tokens likewise; decoding then goes on tensor-parallel.
    # Twice: a short prompt (few rows: all layers delivered in one launch after the read) and a long one (many rows: layer
    # l delivered on a side stream while the read works on layer l + 1).
    import torch
    import torch.distributed as td
    for context, prompt_len in ((32, 12), (320, 160)):
        cfg2 = GptConfig(vocab=cfg.vocab, dim=cfg.dim, heads=cfg.heads, layers=cfg.layers, ff_dim=cfg.ff_dim, context=context)
        w2 = om.make_weights(cfg2, seed=4)
        B4 = 2 * world
        prompt4 = orc.token_ids((B4, prompt_len), 45, cfg2.vocab).astype(np.int32)
        one = GptW8A8(dev, cfg2, w2, B4, max_prefill=prompt_len + 4)
        one.prefill(prompt4)
        dev.synchronize()
        one_pools = one.kv_block.download().view(np.uint16).reshape(cfg2.layers, 2, B4 * one.max_pages, cfg2.heads, one.page_size, cfg2.head_dim)
        one_ids, one_logits = one.read_ids().copy(), one.read_logits().copy()
        m3 = GptW8A8(dev, cfg2, w2, B4, max_prefill=prompt_len + 4, tp_rank=rank, tp_size=world, comm=comm)
        m3.enable_batch_sharded_prefill(w2)
        m3.prefill(prompt4)
        dev.synchronize()
        dist.barrier()
        mine3 = m3.kv_block.download().view(np.uint16).reshape(cfg2.layers, 2, B4 * m3.max_pages, m3.heads_loc, m3.page_size, cfg2.head_dim)
        hl = m3.heads_loc
        assert np.array_equal(mine3, one_pools[:, :, :, rank * hl:(rank + 1) * hl]), "delivered keys / values differ from the one-GPU cache"
        assert mine3.any()
        assert np.array_equal(m3.read_ids(), one_ids), "gathered first tokens differ from the one-GPU model's"
        bl = B4 // world
        assert np.array_equal(m3.replica.read_logits().view(np.uint32), one_logits[rank * bl:(rank + 1) * bl].view(np.uint32))
        got3, _ = m3.generate(prompt4, 10, use_graph=True)
        mine = torch.from_numpy(got3.astype(np.int64))
        ref0 = mine.clone()
        td.broadcast(ref0, 0)
        assert torch.equal(mine, ref0), "ranks disagree on the tokens after a batch-sharded prompt read"
        assert np.array_equal(got3[:, 0], one_ids)
        m3.close()
        one.close()
    dist.barrier()
    print(f"rank {rank}: gpu ok, agreement {agree:.3f}")


def watch_mode():
    """Failure detection between steps, on the host: rank 1 returns after three steps; rank 0 learns of it before it
    queues the fourth (its wait for rank 1's step counter runs out), tears down its (stand-in) communicator and gets
    NS_ERR_COMM.  A second watch shows the other trigger: the transport's own asynchronous error."""
    from nn_b200 import native as N
    rank, world, _ = dist.env_rank()
    dist.broadcast_bytes(b"x" if rank == 0 else None, 1)     # brings the gloo group (and its store) up
    calls = {"abort": 0, "poll": 0}

    def fake_abort():
        calls["abort"] += 1

    def fake_poll():
        calls["poll"] += 1
        return 0

    watch = dist.PeerWatch(rank, world, timeout_s=1.0, comm_error=fake_poll, comm_abort=fake_abort)
    for step in range(3):
        watch.check(step)            # a step of the decoder would be queued here
    if rank == 1:
        print("rank 1: cpu ok (left after three steps)")
        sys.stdout.flush()
        os._exit(0)                  # leaves between steps without a goodbye
    try:
        watch.check(3)
        raise AssertionError("rank 0 must not get past the missing rank")
    except N.NsError as e:
        assert e.code == 5 and "rank 1 did not reach step 3" in e.text, e.text
    assert calls["abort"] == 1 and calls["poll"] > 0
    # the transport reporting an error ends the wait at once
    watch2 = dist.PeerWatch(rank, world, timeout_s=30.0, comm_error=lambda: 6, comm_abort=fake_abort, prefix="ns_watch2")
    import time
    t0 = time.monotonic()
    try:
        watch2.check(0)
        raise AssertionError("an asynchronous transport error must fail the check")
    except N.NsError as e:
        assert e.code == 5 and "error 6" in e.text
    assert time.monotonic() - t0 < 5.0 and calls["abort"] == 2
    print("rank 0: cpu ok (saw rank 1 leave)")
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    {"cpu": cpu_mode, "gpu": gpu_mode, "watch": watch_mode}[sys.argv[1]]()
