"""Generate the golden vectors under tests/golden/ from the reference itself.

Run in a container that has the reference checkout and the installed flashinfer wheel:

    python tests/golden/make_golden.py --reference <path of the reference checkout>

Two fixtures are written (small .npz files, committed):

* ``cache_format.npz`` -- outputs of the reference's own fixture builder
  ``_make_w512_cache`` (tests/test_cute_dsl_mla_fp4.py:56-93).  The function is cut out of
  the reference test file with ``ast`` and executed as is (the file itself cannot be imported:
  its imports need a GPU-only package version).  Pins cache format, quantiser and dequantiser.
* ``attention_fi_reference.npz`` -- outputs of the torch reference that ships inside the
  reference's dependency (flashinfer ``trace/templates/attention.py::_cute_dsl_batch_mla_run_reference``)
  on the dequantised cache, in FP32.  Cross-checks the attention half of the oracle.

Nothing here is used at test time except the .npz files.
"""
from __future__ import annotations

import argparse
import ast
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference_builder(ref_root: Path):
    src = (ref_root / "tests" / "test_cute_dsl_mla_fp4.py").read_text()
    tree = ast.parse(src)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_make_w512_cache")
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"torch": torch, "LATENT_DIM": 512, "ROPE_DIM": 64}
    exec(compile(mod, "reference:_make_w512_cache", "exec"), ns)
    return ns["_make_w512_cache"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    builder = load_reference_builder(Path(args.reference))

    g = torch.Generator().manual_seed(20260101)
    # 3 pages x 16 tokens; include exact ties (multiples of the thresholds) and large values
    source = torch.randn(3, 16, 576, generator=g).to(torch.float16)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 6.0, 7.5, -9.0, 0.0, -0.0, 0.125, 3.0])
    source[0, 0, :16] = ties.to(torch.float16)          # scale 0.5 on token 0
    source[0, 1, :16] = (ties * 1.0).to(torch.float16)  # scale 1.0 on token 1
    fp4_cache, token_scale, fp8_cache = builder(source)
    np.savez_compressed(
        HERE / "cache_format.npz",
        source_f16_bits=source.view(torch.int16).numpy(),
        fp4_cache=fp4_cache.numpy(),
        token_scale=token_scale.numpy(),
        fp8_cache_bits=fp8_cache.view(torch.uint8).numpy(),
    )

    # attention cross-check through the dependency's torch reference, fed FP32 inputs
    from flashinfer.trace.templates.attention import _cute_dsl_batch_mla_run_reference as fi_ref

    g = torch.Generator().manual_seed(20260102)
    B, H, ps, pages_per = 2, 4, 16, 3
    src2 = torch.randn(B * pages_per + 1, ps, 576, generator=g).to(torch.float16)
    cache2, scale2, fp8_2 = builder(src2)
    q = (torch.randn(B, 1, H, 576, generator=g) * 0.5).to(torch.float8_e4m3fn)
    block_tables = torch.tensor([[4, 0, 2], [1, 6, 3]], dtype=torch.int32)
    seq_lens = torch.tensor([41, 17], dtype=torch.int32)
    softmax_scale = 1.0 / 512 ** 0.5
    out = fi_ref(q.float(), fp8_2.float(), block_tables, seq_lens, 48, softmax_scale, 1.25)
    np.savez_compressed(
        HERE / "attention_fi_reference.npz",
        q_bits=q.view(torch.uint8).numpy(),
        fp4_cache=cache2.numpy(),
        token_scale=scale2.numpy(),
        block_tables=block_tables.numpy(),
        seq_lens=seq_lens.numpy(),
        softmax_scale=np.float32(softmax_scale),
        output_scale=np.float32(1.25),
        out=out.numpy(),
    )
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
