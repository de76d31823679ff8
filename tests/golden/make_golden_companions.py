"""Generates tests/golden/golden_companions.npz: batch-statistics BatchNormalization and the backward
passes of BatchNormalization, ReLU, Add2, MaxPooling and GlobalAveragePooling as computed by the
reference's own CPU functions (oracle/_ref/libnnabla_ref.so, built by `make -C oracle ref`).

    python tests/golden/make_golden_companions.py

Inputs are regenerated from tests/companion_cases.py (seeded); only the reference's outputs are stored."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import companion_cases as cc  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    g = {}
    for i in range(len(cc.BN_SHAPES)):
        c = cc.bn_case(i)
        y, m, v, rm, rv = ref.batch_normalization_batch(c["x"], c["beta"], c["gamma"], c["mean"], c["var"])
        for k, a in zip(("y", "m", "v", "rm", "rv"), (y, m, v, rm, rv)):
            g["bn%d/fwd_%s" % (i, k)] = a
        for batch_stat in (True, False):
            for accum in (False, True):
                dx, db, dg = ref.batch_normalization_backward(
                    c["x"], c["beta"], c["gamma"], c["mean"], c["var"], c["dy"], batch_stat=batch_stat,
                    dmean=c["dmean"] if batch_stat else None, dvar=c["dvar"] if batch_stat else None,
                    accum=(accum,) * 3, grads=c["g0"])
                k = "bn%d/bwd_%d%d" % (i, int(batch_stat), int(accum))
                g[k + "_dx"], g[k + "_dbeta"], g[k + "_dgamma"] = dx, db, dg
    for i in range(len(cc.POOL_CASES)):
        c = cc.pool_case(i)
        y = ref.max_pooling(c["x"], c["kernel"], c["stride"], c["ib"], c["pad"])
        dy = c["rng"].randn(*y.shape).astype(np.float32)
        g["pool%d/dy" % i] = dy
        for accum in (False, True):
            g["pool%d/dx_%d" % (i, int(accum))] = ref.max_pooling_backward(c["x"], dy, c["kernel"], c["stride"], c["ib"],
                                                                          c["pad"], accum, c["g0"])
    e = cc.elementwise_case()
    for accum in (False, True):
        g["relu/dx_%d" % accum] = ref.relu_backward(e["x"], e["dy"], accum, e["g0"])
        g["add2/dx_%d" % accum] = ref.add2_backward(e["x"], e["x"][::-1].copy(), e["dy"], (accum, accum),
                                                    (e["g0"], e["g0"]))[1]
        g["gap/dx_%d" % accum] = ref.global_average_pooling_backward(e["x"], e["dyp"], accum, e["g0"])
    out = os.path.join(HERE, "golden_companions.npz")
    np.savez_compressed(out, **g)
    print(out, len(g), "arrays", os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
