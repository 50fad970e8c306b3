#!/usr/bin/env python
"""Records golden vectors from the reference's own CUDA kernels (oracle/_ref/libgemma4_ref.so, built
from the gemma.c sources by oracle/build_ref.sh) on a CUDA device.

    python tests/golden/make_golden.py [output_dir]      # default: tests/golden/_recorded

Writes one small .npz per case of tests/golden_cases.py: the outputs only (prepared q, the appended
cache rows, attention rows, projection rows), plus a digest of the seeded inputs. Copy the files into tests/golden/.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

from oracle import ref_binding as ref  # noqa: E402
from oracle.binding import cache_offset  # noqa: E402
from tests import golden_cases as gc  # noqa: E402
from tests.gpu_util import dev, host_u16  # noqa: E402


def record_append(name, out_dir):
    case = gc.build_append(name)
    cfg = case.cfg
    elems = cfg[0] * cfg[1] * cfg[2] * cfg[5] * cfg[6]
    ck = torch.zeros(elems, dtype=torch.int16, device="cuda")
    cv = torch.zeros(elems, dtype=torch.int16, device="cuda")
    qp = torch.zeros(case.q.shape, dtype=torch.int16, device="cuda")
    rc = ref.decode_append(qp, ck, cv, cfg, dev(case.page_table), dev(case.token_position), case.layer, dev(case.q),
                           dev(case.k), None if case.v is None else dev(case.v), dev(case.q_w), dev(case.k_w), dev(case.cos), dev(case.sin),
                           case.token_position.size)
    torch.cuda.synchronize()
    assert rc == 0, rc
    hk, hv = host_u16(ck), host_u16(cv)
    row = cfg[5] * cfg[6]
    rows_k, rows_v = [], []
    for b, pos in enumerate(case.token_position):
        phys = int(case.page_table[b, (pos // cfg[2]) % cfg[3]])
        base = cache_offset(cfg, case.layer, phys, int(pos % cfg[2]), 0, 0)
        rows_k.append(hk[base:base + row])
        rows_v.append(hv[base:base + row])
    written = int((hk != 0).sum())
    np.savez_compressed(out_dir / f"{name}.npz", q_prepared=host_u16(qp).reshape(case.q.shape),
                        k_rows=np.stack(rows_k), v_rows=np.stack(rows_v), nonzero_k=np.int64(written),
                        digest=np.array(gc.append_digest(case)))
    print(name, "ok")


def record_attention(name, out_dir):
    case, split_size, num_splits = gc.build_attention(name)
    B, H, D = case.batch, case.q_heads, case.head_dim
    out = torch.zeros((B, H, D), dtype=torch.int16, device="cuda")
    rows = B * H * num_splits
    pm = torch.zeros(max(rows, 1), dtype=torch.float32, device="cuda")
    pl = torch.zeros_like(pm)
    pacc = torch.zeros(max(rows, 1) * D, dtype=torch.float32, device="cuda")
    rc = ref.decode_attention(out, pm, pl, pacc, dev(case.q), dev(case.cache_k), dev(case.cache_v),
                              dev(case.page_table), dev(case.seq_lengths), case.cfg, case.layer, case.scale,
                              split_size, num_splits, B)
    torch.cuda.synchronize()
    assert rc == 0, rc
    np.savez_compressed(out_dir / f"{name}.npz", out=host_u16(out).reshape(B, H, D),
                        digest=np.array(gc.attention_digest(case)))
    print(name, "ok")


def record_projection(name, out_dir):
    case = gc.build_projection(name)
    d = {n: dev(case[n]) for n in gc.PROJECTION_INPUTS}
    raw = torch.zeros(case["cols"], dtype=torch.int16, device="cuda")
    scratch = torch.zeros(gc.HIDDEN, dtype=torch.int16, device="cuda")
    rc = ref.decode_ingress(raw, scratch, d["x"], d["w_in"], d["w_qkv"], case["global_geometry"])
    outs = [torch.zeros(gc.HIDDEN, dtype=torch.int16, device="cuda") for _ in range(4)]
    rc2 = ref.decode_egress(*outs, d["attn"], d["w_o"], d["w_post"], d["w_pre"], d["x"], case["global_geometry"])
    torch.cuda.synchronize()
    assert rc == 0 and rc2 == 0, (rc, rc2)
    values = dict(zip(gc.PROJECTION_OUTPUTS, [host_u16(raw)] + [host_u16(t) for t in outs]))
    np.savez_compressed(out_dir / f"{name}.npz", digest=np.array(gc.projection_digest(case)), **values)
    print(name, "ok")


def main():
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else REPO / "tests" / "golden" / "_recorded"
    out_dir.mkdir(parents=True, exist_ok=True)
    assert ref.available(), "oracle/_ref/libgemma4_ref.so is missing: run oracle/build_ref.sh where the sources are"
    for name in gc.APPEND_ALL:
        record_append(name, out_dir)
    for name in gc.ATTENTION_ALL:
        record_attention(name, out_dir)
    if ref.has_projections():
        for name in gc.PROJECTION_ALL:
            record_projection(name, out_dir)


if __name__ == "__main__":
    main()
