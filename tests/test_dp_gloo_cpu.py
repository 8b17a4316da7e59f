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
