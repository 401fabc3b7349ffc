"""Generate the golden fixtures in this directory from the reference's own CUDA extension.

Runs on a machine with a Blackwell GPU and ``oracle/_ref/permuto_ref_C.so`` (built from the
unmodified reference sources by ``oracle/build_ref.py``):

    python tests/golden/make_golden.py --out tests/golden

For every case of ``cases.py`` it stores the reference's outputs (never the inputs, which are
regenerated from seeds): features, table gradient (sparse), position gradient, the two
double-backward outputs, single-point backward probes that reveal the reference's hash slots
and barycentric weights exactly, and the scale factor produced by replaying the reference's
ATen operator sequence.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cases  # noqa: E402
from oracle import ref_shim  # noqa: E402

PROBE_POINTS = 32


def to_rows(t_lfn: torch.Tensor) -> np.ndarray:
    """[L, 2, N] -> [N, 2L] (the module's output order, reference modules.py:87)."""
    return t_lfn.permute(2, 0, 1).reshape(t_lfn.shape[2], -1).contiguous().cpu().numpy()


def to_lfn(rows: np.ndarray) -> torch.Tensor:
    n, w = rows.shape
    return torch.from_numpy(rows).cuda().reshape(n, w // 2, 2).permute(1, 2, 0).contiguous()


def sparse(t: torch.Tensor):
    flat = t.contiguous().reshape(-1)
    idx = torch.nonzero(flat, as_tuple=False).reshape(-1)
    return idx.to(torch.int32).cpu().numpy(), flat[idx].cpu().numpy()


def run_case(name: str) -> dict:
    c = cases.CASES[name]
    inp = cases.make_inputs(name)
    d, cap, nl, n = c["pos_dim"], c["capacity"], c["nr_levels"], c["n"]
    dev = "cuda"
    table = torch.from_numpy(inp["table"]).to(dev)
    shift = torch.from_numpy(inp["shift"]).to(dev)
    pos = torch.from_numpy(inp["positions"]).to(dev)
    anneal = torch.from_numpy(inp["anneal"]).to(dev)
    enc = ref_shim.RefEncoding(d, cap, nl, inp["sigmas"], shift, c.get("concat", False),
                               c.get("points_scaling", 1.0))
    out = {"aten_scale": ref_shim.aten_scale_factor(inp["sigmas"], d).cpu().numpy()}
    out["features"] = to_rows(enc.forward_raw(table, pos, anneal))
    if "backward" in c["parts"]:
        g = to_lfn(inp["grad_out"])
        tg, pg = enc.backward_raw(table, pos, anneal, g, True, True)
        out["table_grad_idx"], out["table_grad_val"] = sparse(tg)
        out["pos_grad"] = pg.contiguous().cpu().numpy()
        # single-point probes: upstream gradient 1 on feature 0 of every level for one point
        k = nl * (d + 1)
        m = min(PROBE_POINTS, n)
        pidx = np.full((m, k), -1, np.int32)
        pval = np.zeros((m, k), np.float32)
        for j in range(m):
            gp = torch.zeros_like(g)
            gp[:nl, 0, j] = 1.0
            tgp, _ = enc.backward_raw(table, pos, anneal, gp, True, False)
            i, v = sparse(tgp)
            assert len(i) <= k
            pidx[j, :len(i)] = i
            pval[j, :len(i)] = v
        out["probe_idx"], out["probe_val"] = pidx, pval
    if "double" in c["parts"]:
        g = to_lfn(inp["grad_out"])
        dpg = torch.from_numpy(inp["dpg"]).to(dev)
        tg2, ggs = enc.double_backward_raw(table, pos, anneal, dpg, g)
        out["dbl_table_grad_idx"], out["dbl_table_grad_val"] = sparse(tg2)
        out["dbl_grad_grad_out"] = to_rows(ggs)
    torch.cuda.synchronize()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    ap.add_argument("--cases", nargs="*", default=sorted(cases.CASES))
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    for name in args.cases:
        res = run_case(name)
        path = os.path.join(args.out, name + ".npz")
        np.savez_compressed(path, **res)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB", {k: v.shape for k, v in res.items()})
    return 0


if __name__ == "__main__":
    sys.exit(main())
