"""Shared helpers of the test suite: golden fixtures, oracle calls, the operator call."""
from __future__ import annotations

import importlib.util
import os
from typing import Dict

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN_DIR = os.path.join(HERE, "golden")

_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN_DIR, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)
GOLDEN_CASES = make_golden.CASES

# Tolerance of the operator against the PyTorch path for bf16 outputs (the build's stated bar;
# the reference itself only asks atol = rtol = 5e-2 of its fp8 kernels, test_pa_mtp.py:785,912).
ATOL, RTOL = 2e-2, 1e-2


def load_golden(name: str) -> Dict:
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = torch.from_numpy(z["out_bf16_bits"].copy()).view(torch.bfloat16)
    return {"out": out, "context_lens": torch.from_numpy(z["context_lens"].copy()),
            "digest": dict(zip(z["digest_keys"].tolist(), z["digest_vals"].tolist())),
            "torch_version": str(z["torch_version"])}


def golden_inputs(name: str):
    from triton_op_b200.inputs import make_inputs
    cfg, seed, dist = GOLDEN_CASES[name]
    return make_inputs(cfg, seed=seed, device="cpu", dist=dist)


def oracle_output(inp) -> torch.Tensor:
    """The oracle on ``inp`` (token-major [S*L, Hq, D] bf16), on inp's device."""
    from oracle import pa_oracle
    ks, vs = inp.flat_scales()
    return pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables,
                                     inp.context_lens, inp.query_indptr(), ks, vs)


def run_operator(inp, partition_size=None, status=None, **kw):
    """Calls the CUDA operator on ``inp`` (already on the GPU); returns (token-major output, dict)."""
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import unpack_mtp
    c = inp.cfg
    out = torch.full_like(inp.query, float("nan"))
    res = paged_attention_decode(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens,
                                 inp.block_tables, inp.softmax_scale, c.query_len, inp.max_context,
                                 torch.bfloat16, None, inp.key_scale, inp.value_scale,
                                 partition_size=partition_size or c.partition_size, status=status, **kw)
    return unpack_mtp(out, c.num_seqs, c.query_len, c.kv_heads), res


def assert_close(actual: torch.Tensor, expected: torch.Tensor, atol=ATOL, rtol=RTOL, what=""):
    a, e = actual.float().cpu(), expected.float().cpu()
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    assert not torch.isnan(a).any(), f"{what}: NaN in the result"
    err = (a - e).abs()
    bad = err > (atol + rtol * e.abs())
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance, "
                           f"max abs err {float(err.max()):.3e}")
    return float(err.max())
