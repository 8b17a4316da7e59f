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
    if shard == "bf16":
        os.environ["ZN_DP_GATHER_BF16"] = "1"      # the sharded update's optional exchange of the bf16 operand copy
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


@pytest.mark.parametrize("shard", [False, True, "bf16"], ids=["replicated", "sharded", "sharded-bf16-exchange"])
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
    if shard == "bf16" and prec_name != "BF16_TC":
        pytest.skip("the bf16 exchange exists for bf16 networks only")
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


def _leaving_rank(rank, world, uid_path, out_dir):
    """Rank 1 leaves after two steps, between steps, with nothing of its own in flight; rank 0 then starts a third
    step whose first all-reduce can never complete and must get ZN_ERR_NCCL from the deadline, not a hang."""
    import time
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import zigneuron_b200 as zn
    prec = zn.Precision.FP32_SIMT
    x, t, Ws, bs = _data("mse")
    be = zn.Backend(rank, prec)
    if rank == 0:
        uid = zn.Backend.dp_unique_id()
        with open(uid_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(uid_path + ".tmp", uid_path)
    else:
        for _ in range(600):
            if os.path.exists(uid_path):
                break
            time.sleep(0.05)
        uid = open(uid_path, "rb").read()
    be.dp_init(rank, world, uid)
    be.dp_set_timeout_ms(3000)
    net = _build(zn, be, prec, Ws, bs, False)
    net.setDataParallel(B)
    lo, hi = zn.Backend.distributeWorkload(B, world, rank)
    for _ in range(2):
        net.trainStep(x[lo:hi], t[lo:hi], LR, zn.Loss.mse)
    be.endCommandBatch()                       # every lane of this rank is idle
    gone = os.path.join(out_dir, "rank1_gone")
    if rank == 1:
        net.deinit()
        be.deinit()
        open(gone, "w").close()
        return
    for _ in range(1200):                      # the survivor learns nothing on the host: it just takes the next step
        if os.path.exists(gone):
            break
        time.sleep(0.05)
    result = {}
    t0 = time.perf_counter()
    try:
        net.trainStep(x[lo:hi], t[lo:hi], LR, zn.Loss.mse)
        result["first"] = 0
    except zn.ZnError as e:
        result["first"], result["text"] = e.status, str(e)
    result["seconds"] = time.perf_counter() - t0
    try:
        net.trainStep(x[lo:hi], t[lo:hi], LR, zn.Loss.mse)
        result["second"] = 0
    except zn.ZnError as e:
        result["second"] = e.status
    np.savez(os.path.join(out_dir, "survivor.npz"), first=result["first"], second=result["second"],
             seconds=result["seconds"], text=result.get("text", ""))
    net.deinit()
    be.deinit()


def test_survivor_of_a_lost_rank_gets_an_error_not_a_hang(tmp_path):
    import zigneuron_b200 as zn
    if zn.Backend.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_leaving_rank, args=(2, str(tmp_path / "uid"), str(tmp_path)), nprocs=2, join=True)
    r = np.load(tmp_path / "survivor.npz")
    assert int(r["first"]) == 10, str(r["text"])          # ZN_ERR_NCCL
    assert "aborted" in str(r["text"])
    assert 2.5 <= float(r["seconds"]) <= 20.0               # the 3 s deadline, not the 120 s default
    assert int(r["second"]) == 10                            # the communicator stays refused until re-initialised


# ---- config 4 at full width: 4096-8192-8192-8192-4096, bf16, Adam, global batch 2 x 1024 -------------------------

WIDE_STEPS, WIDE_ROWS, WIDE_STRIDE = 2, 2048, 4099


def _wide_setup(zn, be):
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import configs as cfg
    net = zn.Network(be, zn.Precision.BF16_TC)
    for i, ((a, b), act) in enumerate(zip(cfg.WIDE_DIMS, cfg.WIDE_ACTS)):
        net.addDense(a, b, act)
        net.setWeights(i, cfg.wide_layer_weights(i, seed=3), np.zeros(b, np.float32))
    net.setOptimizer(zn.Adam(beta1=0.9, beta2=0.999, eps=1e-8))
    x, t = cfg.wide_rows(WIDE_ROWS, seed=3)
    return net, x, t


def _wide_summary(net, losses):
    import hashlib
    out = {"losses": np.array(losses, np.float32)}
    for i in range(4):
        W, b = net.getWeights(i)
        gW, gb = net.getGrads(i)
        out[f"hash{i}"] = np.frombuffer(hashlib.sha256(W.tobytes() + b.tobytes()).digest(), np.uint8)
        out[f"W{i}"], out[f"gW{i}"], out[f"gb{i}"] = W.ravel()[::WIDE_STRIDE].copy(), gW.ravel()[::WIDE_STRIDE].copy(), gb
    return out


def _wide_rank(rank, world, uid_path, out_dir):
    import time
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import zigneuron_b200 as zn
    be = zn.Backend(rank, zn.Precision.BF16_TC)
    if rank == 0:
        uid = zn.Backend.dp_unique_id()
        with open(uid_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(uid_path + ".tmp", uid_path)
    else:
        for _ in range(1200):
            if os.path.exists(uid_path):
                break
            time.sleep(0.05)
        uid = open(uid_path, "rb").read()
    be.dp_init(rank, world, uid)
    net, x, t = _wide_setup(zn, be)
    net.setDataParallel(WIDE_ROWS)
    lo, hi = zn.Backend.distributeWorkload(WIDE_ROWS, world, rank)
    losses = [net.trainStep(np.ascontiguousarray(x[lo:hi]), np.ascontiguousarray(t[lo:hi]), 1e-3, zn.Loss.mse)
              for _ in range(WIDE_STEPS)]
    np.savez(os.path.join(out_dir, f"wide{rank}.npz"), **_wide_summary(net, losses))
    net.deinit()          # between steps, nothing in flight
    be.deinit()


def test_two_gpus_at_full_width_match_one_gpu(tmp_path):
    """Config 4's network at its stated width on two ranks of 1024 rows each: both ranks end bit-identical, and
    losses, summed gradients and updated weights agree with one GPU taking all 2048 rows."""
    import zigneuron_b200 as zn
    if zn.Backend.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from util import rel_l2
    mp.spawn(_wide_rank, args=(2, str(tmp_path / "uid"), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "wide0.npz"), np.load(tmp_path / "wide1.npz")
    assert np.array_equal(r0["losses"], r1["losses"])
    for i in range(4):
        assert np.array_equal(r0[f"hash{i}"], r1[f"hash{i}"]), f"layer {i} differs between the ranks"
    be = zn.Backend(0, zn.Precision.BF16_TC)
    net, x, t = _wide_setup(zn, be)
    one = _wide_summary(net, [net.trainStep(x, t, 1e-3, zn.Loss.mse) for _ in range(WIDE_STEPS)])
    print(f"\nconfig4 full width, 2 ranks x 1024 rows: losses {r0['losses']} one GPU {one['losses']}")
    assert np.allclose(r0["losses"], one["losses"], rtol=1e-4)
    for i in range(4):
        dg, db, dw = rel_l2(r0[f"gW{i}"], one[f"gW{i}"]), rel_l2(r0[f"gb{i}"], one[f"gb{i}"]), rel_l2(r0[f"W{i}"], one[f"W{i}"])
        print(f"  layer {i}: gW {dg:.3e} gb {db:.3e} W {dw:.3e}")
        assert dg <= 2e-2 and db <= 2e-2 and dw <= 2e-2
    net.deinit()
    be.deinit()
