"""Data-parallel arithmetic on CPU ranks (gloo, world size 2): shard rows with the
reference's round-robin split, compute shard gradients with the oracle, sum them
with an all-reduce, clip and update -- and compare with the oracle run on the whole
batch in one process.  This is the host-side contract the NCCL path implements."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _build(loss, adam):
    from oracle import zn_oracle as zo
    from util import reference_init
    rng = np.random.default_rng(11)
    net = zo.Net()
    dims = [(6, 16, zo.RELU, "relu"), (16, 8, zo.RELU, "relu"), (8, 4, zo.LINEAR, "linear")]
    for i, (a, b, act, name) in enumerate(dims):
        net.add_dense(a, b, act)
        net.set_params(i, reference_init(rng, a, b, name), rng.uniform(-0.1, 0.1, b).astype(np.float32))
        if adam:
            net.set_adam(i)
    B = 37   # odd on purpose: shards of 19 and 18 rows
    x = rng.standard_normal((B, 6)).astype(np.float32)
    if loss == zo.MSE:
        t = rng.standard_normal((B, 4)).astype(np.float32)
    else:
        t = np.eye(4, dtype=np.float32)[rng.integers(0, 4, B)]
    return net, x, t


def _rank(rank, world, port, loss, adam, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import zn_oracle as zo
    net, x, t = _build(loss, adam)
    B = x.shape[0]
    losses = []
    for step in range(3):
        lo, hi = zo.distribute_round_robin(B, world, rank)
        shard_loss = net.shard_gradients(x[lo:hi], t[lo:hi], hi - lo, B, loss)
        tot = torch.tensor([shard_loss], dtype=torch.float32)
        dist.all_reduce(tot)
        for i in range(3):
            gW, gb = net.get_grads(i)
            flat = torch.from_numpy(np.concatenate([gW.ravel(), gb]))
            dist.all_reduce(flat)                     # sum, not mean: the reference's gradients carry no 1/B
            flat = flat.numpy()
            net.set_grads(i, flat[:gW.size].reshape(gW.shape), flat[gW.size:])
        net.clip_and_update(0.05)
        losses.append(float(tot) if loss == zo.MSE else float(tot) / B)
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), losses=np.array(losses, np.float32),
             **{f"W{i}": net.get_params(i)[0] for i in range(3)}, **{f"b{i}": net.get_params(i)[1] for i in range(3)})
    dist.destroy_process_group()


@pytest.mark.parametrize("loss_name,adam", [("mse", False), ("ce", True)])
def test_two_rank_sum_equals_single_process(tmp_path, loss_name, adam):
    from oracle import zn_oracle as zo
    loss = zo.MSE if loss_name == "mse" else zo.CE_LOGITS
    port = 29400 + (os.getpid() % 400) + (0 if adam else 1)
    mp.spawn(_rank, args=(2, port, loss, adam, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    net, x, t = _build(loss, adam)
    want = [net.train_step(x, t, x.shape[0], 0.05, loss) for _ in range(3)]
    assert np.allclose(r0["losses"], want, rtol=2e-5, atol=1e-6)
    for i in range(3):
        W, b = net.get_params(i)
        # both ranks hold identical parameters, equal to the single-process run up to summation order
        assert np.array_equal(r0[f"W{i}"], r1[f"W{i}"]) and np.array_equal(r0[f"b{i}"], r1[f"b{i}"])
        assert np.allclose(r0[f"W{i}"], W, rtol=1e-4, atol=2e-6)
        assert np.allclose(r0[f"b{i}"], b, rtol=1e-4, atol=2e-6)


def _rank_sharded(rank, world, port, loss, adam, out_dir):
    """The sharded update the library offers under data parallel, restated with the oracle's flat update functions:
    reduce-scatter of each layer's [W | pad | b] block, sums of squares of the own piece, one all-reduce of
    L + 1 doubles (squares and loss), update of the own piece, all-gather."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import zn_oracle as zo
    net, x, t = _build(loss, adam)
    B, L, lr = x.shape[0], 3, np.float32(0.05)
    up4 = lambda v: (v + 3) // 4 * 4
    state = [None] * L
    losses = []
    for step in range(3):
        lo_r, hi_r = zo.distribute_round_robin(B, world, rank)
        shard_loss = net.shard_gradients(x[lo_r:hi_r], t[lo_r:hi_r], hi_r - lo_r, B, loss)
        scal = np.zeros(L + 1, np.float64)
        scal[L] = shard_loss
        pieces = []
        for i in range(L):
            (W, b), (gW, gb) = net.get_params(i), net.get_grads(i)
            b_off = up4(W.size)
            blk = up4(b_off + b.size)
            shard = up4((blk + world - 1) // world)
            g = np.zeros(world * shard, np.float32)
            g[:W.size], g[b_off:b_off + b.size] = gW.ravel(), gb
            gt = torch.from_numpy(g)
            dist.all_reduce(gt)                               # gloo has no reduce-scatter: sum, then keep the own piece
            lo, hi = rank * shard, (rank + 1) * shard
            own = g[lo:hi].copy()
            scal[i] = float((own.astype(np.float64) ** 2).sum())
            pieces.append((W, b, b_off, shard, lo, hi, own))
        st = torch.from_numpy(scal)
        dist.all_reduce(st)
        norm = np.float32(np.sqrt(np.float32(scal[:L].sum())))
        factor = np.float32(1.0) / (norm + np.float32(1e-6)) if norm > 1.0 else np.float32(1.0)
        for i, (W, b, b_off, shard, lo, hi, own) in enumerate(pieces):
            p = np.zeros(world * shard, np.float32)
            p[:W.size], p[b_off:b_off + b.size] = W.ravel(), b
            own = own * factor if factor != 1.0 else own
            if adam and state[i] is None:
                state[i] = [np.zeros(world * shard, np.float32), np.zeros(world * shard, np.float32), 0]
            if adam:
                state[i][2] += 1
                bc1, bc2 = zo.adam_bias_corrections(0.9, 0.999, state[i][2])
            for part, (r0_, r1_) in enumerate([(0, W.size), (b_off, b_off + b.size)]):
                a0, a1 = max(lo, r0_), min(hi, r1_)
                if a0 >= a1:
                    continue
                gp = own[a0 - lo:a1 - lo]
                if adam:
                    m, v = state[i][0], state[i][1]
                    p[a0:a1], m[a0:a1], v[a0:a1] = zo.adam_update(p[a0:a1], gp, m[a0:a1], v[a0:a1], lr, 0.9, 0.999, 1e-8, bc1, bc2)
                elif part == 0:
                    p[a0:a1] = zo.sgd_update(p[a0:a1], gp, lr, 0.0)
                else:
                    p[a0:a1] = zo.sgd_update_bias(p[a0:a1], gp, lr)
            mine = torch.from_numpy(p[lo:hi].copy())
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            p = torch.cat(parts).numpy()
            net.set_params(i, p[:W.size].reshape(W.shape), p[b_off:b_off + b.size])
        losses.append(float(scal[L]) if loss == zo.MSE else float(scal[L]) / B)
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), losses=np.array(losses, np.float32),
             **{f"W{i}": net.get_params(i)[0] for i in range(3)}, **{f"b{i}": net.get_params(i)[1] for i in range(3)})
    dist.destroy_process_group()


@pytest.mark.parametrize("loss_name,adam", [("mse", False), ("ce", True)])
def test_sharded_update_equals_single_process(tmp_path, loss_name, adam):
    from oracle import zn_oracle as zo
    loss = zo.MSE if loss_name == "mse" else zo.CE_LOGITS
    port = 29800 + (os.getpid() % 150) + (0 if adam else 1)
    mp.spawn(_rank_sharded, args=(2, port, loss, adam, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    net, x, t = _build(loss, adam)
    want = [net.train_step(x, t, x.shape[0], 0.05, loss) for _ in range(3)]
    assert np.allclose(r0["losses"], want, rtol=2e-5, atol=1e-6)
    for i in range(3):
        W, b = net.get_params(i)
        assert np.array_equal(r0[f"W{i}"], r1[f"W{i}"]) and np.array_equal(r0[f"b{i}"], r1[f"b{i}"])
        assert np.allclose(r0[f"W{i}"], W, rtol=1e-4, atol=2e-6)
        assert np.allclose(r0[f"b{i}"], b, rtol=1e-4, atol=2e-6)
