"""Generates tests/golden/triton_*.npz by RUNNING the reference's plain-Triton split-KV decode
(pa_decode_triton.py:523-685 of a yanguahe/triton_op checkout) on CPU under the Triton interpreter:

    TRITON_INTERPRET=1 python tests/golden/make_golden_triton.py /path/to/yanguahe_triton_op

That entry point takes ``alibi_slopes`` and returns the split-KV intermediates (``tmp_output``,
``exp_sums``, ``max_logits``) beside the output, so these fixtures pin what the reference's own
PyTorch path cannot: the ALiBi bias and the per-partition (max, sum, normalised output) triples.
The module imports ``aiter.test_common.perftest`` (AMD's package, absent here) only to time its
launches; a pass-through stand-in of that decorator is registered before the import.  The
interpreter has no bf16, so the reference runs on fp16 copies of the bf16 inputs (the same values:
every bf16 number of these magnitudes is an fp16 number) with ``tl.float16`` as compute type.
Inputs come from ``triton_op_b200.inputs.make_inputs`` with a fixed seed; a fixture stores
outputs, slopes and a SHA-256 of every input.  Nothing of the reference's source is written out.
"""
from __future__ import annotations

import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from triton_op_b200.inputs import DecodeConfig, make_inputs  # noqa: E402
from make_golden import input_digest  # noqa: E402

# name -> (config, seed, context lengths, with ALiBi)
_G4 = DecodeConfig("triton_g4", 3, 8, 2, 16, 1, ("fixed", 1), kv_dtype="bf16", quant="none")
_G16 = DecodeConfig("triton_g16", 2, 16, 1, 16, 1, ("fixed", 1), kv_dtype="bf16", quant="none")
CASES = {
    "triton_g4": (_G4, 11, [300, 513, 77], False),
    "triton_g4_alibi": (_G4, 11, [300, 513, 77], True),
    "triton_g16": (_G16, 12, [260, 600], False),
    "triton_g16_alibi": (_G16, 12, [260, 600], True),
}


def alibi_slopes_for(num_heads: int) -> torch.Tensor:
    """The usual geometric slopes 2^(-8 i / n), i = 1..n."""
    return 2.0 ** (-8.0 * torch.arange(1, num_heads + 1, dtype=torch.float32) / num_heads)


def case_inputs(name: str):
    cfg, seed, lens, alibi = CASES[name]
    inp = make_inputs(cfg, seed=seed, device="cpu", context_lens=torch.tensor(lens, dtype=torch.int32))
    return inp, (alibi_slopes_for(cfg.q_heads) if alibi else None)


def load_reference_entry(ref_root: str):
    aiter = types.ModuleType("aiter")
    test_common = types.ModuleType("aiter.test_common")

    def perftest(*_a, **_k):          # the reference wraps its launches in this timer: (result, time)
        def deco(fn):
            def wrapped(*args, **kw):
                return fn(*args, **kw), 0.0
            return wrapped
        return deco

    test_common.perftest = perftest
    aiter.test_common = test_common
    sys.modules.setdefault("aiter", aiter)
    sys.modules.setdefault("aiter.test_common", test_common)
    sys.path.insert(0, ref_root)
    import pa_decode_triton  # noqa: E402  (the reference's module, imported from where it lies)
    import triton.language as tl
    return pa_decode_triton.paged_attention_decode, tl.float16


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden_triton.py <yanguahe/triton_op checkout>")
    entry, compute_type = load_reference_entry(sys.argv[1])
    torch.set_num_threads(1)
    for name in CASES:
        inp, slopes = case_inputs(name)
        q = inp.query.to(torch.float16)
        out = torch.zeros_like(q)
        res = entry(out, q, inp.key_cache.to(torch.float16), inp.value_cache.to(torch.float16), inp.context_lens,
                    inp.block_tables, inp.softmax_scale, inp.max_context, compute_type,
                    torch.tensor(1.0), torch.tensor(1.0), 0, slopes)
        dig = input_digest(inp)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            out=out.float().numpy(), tmp_output=res["tmp_output"].float().numpy(),
            exp_sums=res["exp_sums"].numpy(), max_logits=res["max_logits"].numpy(),
            alibi_slopes=(slopes.numpy() if slopes is not None else np.zeros(0, dtype=np.float32)),
            context_lens=inp.context_lens.numpy(), torch_version=np.array(torch.__version__),
            digest_keys=np.array(list(dig.keys())), digest_vals=np.array(list(dig.values())),
        )
        print(name, tuple(out.shape), float(out.float().abs().mean()), tuple(res["tmp_output"].shape))


if __name__ == "__main__":
    main()
