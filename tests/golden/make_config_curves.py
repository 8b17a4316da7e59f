"""Writes tests/golden/config_curves.json: what the oracle (oracle/zn_oracle.c, the restatement of the reference's
CPU Dense path) computes on configurations 1 and 2 at the step counts the configurations state.

    python tests/golden/make_config_curves.py          # about five minutes on one core

Config 1 (4-20-10-3, cross-entropy with logits, SGD lr 0.005): the loss, gradient norm and clip factor of each of
1000 full-batch steps, and the epoch losses of 20 epochs of the per-sample Network.train loop, with the weights
after each.  Config 2 (784-512-256-10, batch 1024, Adam lr 1e-3): loss, norm and clip factor of each of 100 steps
and a fixed sample of 64 weights per layer (plus the 10 output biases) after steps 1, 2, 5, 10, 20, 50 and 100.
The oracle needs 2.5 s per step of config 2; the GPU tests read these numbers instead of re-running it, and
tests/test_oracle_golden.py re-runs the first steps on the CPU to pin the file to the oracle."""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import zn_oracle as zo   # noqa: E402
import configs as cfg                # noqa: E402


def f32list(a):
    return [float(v) for v in np.asarray(a, np.float32).ravel()]


def oracle_net(dims, acts, Ws, bs, adam):
    net = zo.Net()
    for i, ((a, b), act) in enumerate(zip(dims, acts)):
        net.add_dense(a, b, zo.RELU if act == "relu" else zo.LINEAR)
        net.set_params(i, Ws[i], bs[i])
        if adam:
            net.set_adam(i)
    return net


def snapshot(net, layers):
    out = []
    for i in range(layers):
        W, b = net.get_params(i)
        out.append({"w": f32list(W.ravel()[cfg.snapshot_indices(W.size)]), "b": f32list(b[:10])})
    return out


def main():
    doc = {"_comment": "written by tests/golden/make_config_curves.py from the oracle; see that file"}
    # ---- config 1
    x, t, Ws, bs = cfg.iris_config()
    net = oracle_net(cfg.IRIS_DIMS, cfg.IRIS_ACTS, Ws, bs, False)
    losses, norms, factors = [], [], []
    for _ in range(1000):
        losses.append(net.train_step(x, t, 150, 0.005, zo.CE_LOGITS))
        n, f = net.last_clip()
        norms.append(n)
        factors.append(f)
    c1 = {"full_batch": {"loss": f32list(losses), "norm": f32list(norms), "factor": f32list(factors),
                         "weights": [{"w": f32list(net.get_params(i)[0]), "b": f32list(net.get_params(i)[1])} for i in range(3)]}}
    net = oracle_net(cfg.IRIS_DIMS, cfg.IRIS_ACTS, Ws, bs, False)
    epoch_losses = net.train(x, t, 20, 0.005, zo.CE_LOGITS)
    c1["per_sample"] = {"epoch_loss": f32list(epoch_losses),
                        "weights": [{"w": f32list(net.get_params(i)[0]), "b": f32list(net.get_params(i)[1])} for i in range(3)]}
    doc["config1"] = c1
    # ---- config 2
    x, t, Ws, bs = cfg.mlp784_config()
    net = oracle_net(cfg.MLP784_DIMS, cfg.MLP784_ACTS, Ws, bs, True)
    losses, norms, factors, snaps = [], [], [], {}
    for step in range(1, 101):
        losses.append(net.train_step(x, t, 1024, 1e-3, zo.CE_LOGITS))
        n, f = net.last_clip()
        norms.append(n)
        factors.append(f)
        if step in cfg.SNAP_STEPS:
            snaps[str(step)] = snapshot(net, 3)
        print(step, losses[-1], flush=True)
    doc["config2"] = {"loss": f32list(losses), "norm": f32list(norms), "factor": f32list(factors), "snapshots": snaps}
    with open(os.path.join(HERE, "config_curves.json"), "w") as f:
        json.dump(doc, f)
        f.write("\n")


if __name__ == "__main__":
    main()
