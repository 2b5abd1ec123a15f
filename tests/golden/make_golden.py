"""Generates tests/golden/*.npz from the reference checkout (run where it is mounted):

    python tests/golden/make_golden.py /path/to/yanguahe_triton_op

The two functions of the reference's pure-PyTorch path (``reference_masked_attention`` and
``torch_mha_extend``, test_pa_mtp.py:175-291) are extracted from the file by their AST nodes
and executed on CPU -- the module itself cannot be imported (it needs AMD's ``aiter`` package
and sets the default device to CUDA).  Inputs come from ``triton_op_b200.inputs.make_inputs``
with a fixed seed; a fixture stores the outputs, the context lengths and a SHA-256 of every
input tensor so that a test can tell "the oracle drifted" from "the RNG drifted".
Nothing from the reference's source is written into the fixtures or this repository.
"""
from __future__ import annotations

import ast
import hashlib
import os
import sys
from typing import Dict, List, Optional, Tuple, Union

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from triton_op_b200.inputs import DecodeConfig, make_inputs  # noqa: E402

# name -> (config, seed, dist).  Small enough for the CPU path to finish in seconds.
CASES = {
    "cfg1_small": (DecodeConfig("cfg1_small", 4, 8, 1, 16, 1, ("uniform", 1, 512), pool_blocks=128), 0, "normal"),
    "gqa4_ragged": (DecodeConfig("gqa4_ragged", 6, 32, 8, 16, 1, ("uniform", 1, 700), pool_blocks=400), 1, "normal"),
    "mtp2_g8": (DecodeConfig("mtp2_g8", 5, 8, 1, 16, 2, ("uniform", 2, 600)), 2, "normal"),
    "mtp4_g2_pertoken": (DecodeConfig("mtp4_g2_pertoken", 3, 4, 2, 16, 4, ("uniform", 4, 520), quant="per_token"), 3, "normal"),
    "pertoken_g8": (DecodeConfig("pertoken_g8", 4, 16, 2, 16, 1, ("uniform", 1, 512), quant="per_token"), 4, "normal"),
    "bs64_g5": (DecodeConfig("bs64_g5", 4, 5, 1, 64, 1, ("uniform", 1, 600)), 5, "uniform"),
    "bs1024_mtp2_pertoken": (DecodeConfig("bs1024_mtp2_pertoken", 3, 16, 2, 1024, 2, ("uniform", 900, 2300), quant="per_token"), 6, "normal"),
    "bf16_kv": (DecodeConfig("bf16_kv", 4, 32, 8, 16, 1, ("uniform", 1, 512), kv_dtype="bf16", quant="none"), 7, "normal"),
    "ref_matrix_ctx4097": (DecodeConfig("ref_matrix_ctx4097", 2, 10, 1, 16, 3, ("fixed", 4097)), 8, "uniform"),
    "partition512": (DecodeConfig("partition512", 2, 8, 1, 16, 1, ("cycle", [1500, 2049]), partition_size=512), 9, "normal"),
}


def load_reference_functions(ref_root: str):
    src = open(os.path.join(ref_root, "test_pa_mtp.py")).read()
    tree = ast.parse(src)
    want = {"reference_masked_attention", "torch_mha_extend"}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in want]
    assert {n.name for n in body} == want
    ns = {"torch": torch, "Optional": Optional, "Tuple": Tuple, "List": List, "Dict": Dict, "Union": Union}
    exec(compile(ast.Module(body=body, type_ignores=[]), "test_pa_mtp.py", "exec"), ns)
    return ns["torch_mha_extend"]


def sha(t: Optional[torch.Tensor]) -> str:
    if t is None:
        return "none"
    raw = t.detach().cpu().contiguous()
    raw = raw.view(torch.uint8) if raw.dim() else raw.reshape(1).view(torch.uint8)
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def input_digest(inp) -> Dict[str, str]:
    return {k: sha(getattr(inp, k)) for k in
            ("query_tokens", "key_cache", "value_cache", "key_scale", "value_scale", "block_tables", "context_lens")}


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a yanguahe/triton_op checkout>")
    ref_root = sys.argv[1]
    torch_mha_extend = load_reference_functions(ref_root)
    torch.set_num_threads(1)  # reduction order of the CPU kernels must not depend on the host
    for name, (cfg, seed, dist) in CASES.items():
        inp = make_inputs(cfg, seed=seed, device="cpu", dist=dist)
        ks, vs = inp.flat_scales()
        out = torch_mha_extend(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables,
                               inp.context_lens, inp.query_indptr(), ks, vs)
        dig = input_digest(inp)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            out_bf16_bits=out.contiguous().view(torch.int16).numpy(),
            context_lens=inp.context_lens.numpy(),
            seed=np.int64(seed), dist=np.array(dist),
            torch_version=np.array(torch.__version__),
            digest_keys=np.array(list(dig.keys())), digest_vals=np.array(list(dig.values())),
        )
        print(name, tuple(out.shape), "ctx", inp.context_lens.tolist()[:8], float(out.float().abs().mean()))


if __name__ == "__main__":
    main()
