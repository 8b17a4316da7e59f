"""Data-parallel training on real GPUs: two ranks (one process per GPU, NCCL all-reduce per layer) against
one GPU on the whole batch and against the oracle.  Needs two devices; skipped otherwise.  The ranks leave
only between steps and nothing here faults, traps or hangs a device."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

pytestmark = pytest.mark.gpu

DIMS, ACTS = [(64, 128), (128, 96), (96, 32)], ["relu", "relu", "linear"]
B, STEPS, LR = 200, 4, 0.05


def _data(loss_name):
    from util import reference_init
    rng = np.random.default_rng(17)
    x = rng.standard_normal((B, 64)).astype(np.float32)
    if loss_name == "mse":
        t = rng.standard_normal((B, 32)).astype(np.float32)
    else:
        t = np.eye(32, dtype=np.float32)[rng.integers(0, 32, B)]
    Ws = [reference_init(rng, a, b, act) for (a, b), act in zip(DIMS, ACTS)]
    bs = [rng.uniform(-0.1, 0.1, b).astype(np.float32) for _, b in DIMS]
    return x, t, Ws, bs


def _build(zn, be, prec, Ws, bs, adam):
    net = zn.Network(be, prec)
    for i, ((a, b), act) in enumerate(zip(DIMS, ACTS)):
        net.addDense(a, b, act)
        net.setWeights(i, Ws[i], bs[i])
    if adam:
        net.setOptimizer(zn.Adam())
    return net


def _rank(rank, world, uid_path, out_dir, loss_name, adam, prec_value, shard=False):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    # the last GEMM of a data-parallel step runs its first rows on fewer SMs: 64 of each rank's 100 rows here,
    # so that both of its launches are exercised
    os.environ.setdefault("ZN_DP_RESERVE_ROWS", "64")
    import zigneuron_b200 as zn
    prec = zn.Precision(prec_value)
    loss = zn.Loss.mse if loss_name == "mse" else zn.Loss.cross_entropy_logits
    x, t, Ws, bs = _data(loss_name)
    be = zn.Backend(rank, prec)
    if rank == 0:
        uid = zn.Backend.dp_unique_id()
        with open(uid_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(uid_path + ".tmp", uid_path)
    else:
        import time
        for _ in range(600):
            if os.path.exists(uid_path):
                break
            time.sleep(0.05)
        uid = open(uid_path, "rb").read()
    be.dp_init(rank, world, uid)
    net = _build(zn, be, prec, Ws, bs, adam)
    net.setDataParallel(B)
    if shard:
        net.setUpdateSharding(True)
    lo, hi = zn.Backend.distributeWorkload(B, world, rank)
    losses = [net.trainStep(x[lo:hi], t[lo:hi], LR, loss) for _ in range(STEPS)]
    out = {"losses": np.array(losses, np.float32), "gx": net.getInputGrad(hi - lo)}
    for i in range(len(DIMS)):
        W, b = net.getWeights(i)
        out[f"W{i}"], out[f"b{i}"] = W, b
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), **out)
    net.deinit()
    be.deinit()


@pytest.mark.parametrize("shard", [False, True], ids=["replicated", "sharded"])
@pytest.mark.parametrize("loss_name,adam,prec_name,tol", [("mse", False, "FP32_SIMT", 1e-5), ("ce", True, "FP32_SIMT", 2e-3),
                                                           ("mse", False, "BF16_TC", 2e-2), ("mse", True, "BF16_TC", 2e-2)])
def test_two_gpus_match_one_gpu_and_oracle(tmp_path, loss_name, adam, prec_name, tol, shard):
    import zigneuron_b200 as zn
    if zn.Backend.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from oracle import zn_oracle as zo
    from util import rel_l2
    prec = zn.Precision[prec_name]
    mp.spawn(_rank, args=(2, str(tmp_path / "uid"), str(tmp_path), loss_name, adam, int(prec), shard), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "r0.npz"), np.load(tmp_path / "r1.npz")
    # both ranks end with identical parameters and report the same (global) loss
    assert np.array_equal(r0["losses"], r1["losses"])
    for i in range(len(DIMS)):
        assert np.array_equal(r0[f"W{i}"], r1[f"W{i}"]) and np.array_equal(r0[f"b{i}"], r1[f"b{i}"])
    # one GPU on the whole batch
    x, t, Ws, bs = _data(loss_name)
    loss = zn.Loss.mse if loss_name == "mse" else zn.Loss.cross_entropy_logits
    be = zn.Backend(0, prec)
    net = _build(zn, be, prec, Ws, bs, adam)
    one = [net.trainStep(x, t, LR, loss) for _ in range(STEPS)]
    assert np.allclose(r0["losses"], one, rtol=max(tol, 1e-5), atol=1e-6)
    # the input gradient of the last step: each rank holds the rows of its shard (CE gradients carry no 1/B and
    # MSE uses the global divisor, so the shards are the rows of the one-GPU result)
    gx = net.getInputGrad(B)
    assert rel_l2(np.concatenate([r0["gx"], r1["gx"]]), gx) <= max(tol, 1e-5)
    for i in range(len(DIMS)):
        assert rel_l2(r0[f"W{i}"], net.getWeights(i)[0]) <= tol
    net.deinit()
    be.deinit()
    # the oracle on the whole batch
    onet = zo.Net()
    for i, ((a, b), act) in enumerate(zip(DIMS, ACTS)):
        onet.add_dense(a, b, zo.RELU if act == "relu" else zo.LINEAR)
        onet.set_params(i, Ws[i], bs[i])
        if adam:
            onet.set_adam(i)
    want = [onet.train_step(x, t, B, LR, zo.MSE if loss_name == "mse" else zo.CE_LOGITS) for _ in range(STEPS)]
    assert np.allclose(r0["losses"], want, rtol=max(tol, 2e-5), atol=1e-6)
    for i in range(len(DIMS)):
        if adam and prec_name == "BF16_TC":
            # Adam turns bf16-sized gradient differences into steps of about lr; at lr 0.05 only the bound that
            # Adam itself implies is meaningful against the fp32 oracle (the one-GPU bf16 run above is matched)
            assert np.abs(r0[f"W{i}"] - onet.get_params(i)[0]).max() <= 2.2 * STEPS * LR
        else:
            assert rel_l2(r0[f"W{i}"], onet.get_params(i)[0]) <= tol
