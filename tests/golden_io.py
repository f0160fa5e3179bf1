"""Loads the fixtures of tests/golden/ into the oracle's plain-array containers."""
import os

import numpy as np

from oracle.nq_oracle import ExpertPlanes, ProjPlanes

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def proj_from(z, prefix) -> ProjPlanes:
    N, K, nm, rk, bk = (int(v) for v in z[prefix + "meta"])
    fl, var = z[prefix + "flags"], z[prefix + "var"]
    return ProjPlanes(N=N, K=K, base=z[prefix + "base"].view(np.uint8), p4=z[prefix + "p4"].view(np.uint8),
                      d4=z[prefix + "d4"].view(np.uint32), flags=fl.view(np.uint64) if fl.size else None,
                      var=var if var.size else None, nm=max(nm, 0), rk=rk, bk=bk)


def expert_from(z, prefix, H, I) -> ExpertPlanes:
    ex = ExpertPlanes(H=H, I=I, gu=proj_from(z, prefix + "gu."), dn=proj_from(z, prefix + "dn."),
                      scales=z[prefix + "scales"], had_dn=int(z[prefix + "had_dn"][0]))
    if prefix + "lr" in z.files:
        ex.lr, ex.lr4 = z[prefix + "lr"], z[prefix + "lr4"]
        ex.rg, ex.rd = (int(v) for v in z[prefix + "r"])
    return ex


def layer_from(name):
    z = load(name)
    H, I, E, topk, B = (int(v) for v in z["shape"])
    levels = [int(v) for v in z["levels"]]
    experts = [expert_from(z, f"e{e}.", H, I) if f"e{e}.scales" in z.files else None for e in range(E)]
    return dict(H=H, I=I, E=E, topk=topk, B=B, levels=levels, experts=experts, x=z["x"].view(np.float16),
                sel=z["sel"], rw=z["rw"].view(np.float16), out=z["out"])
