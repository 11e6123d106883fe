"""Generates tests/golden/quant_torch_ref.npz from the REFERENCE's independent torch statement of the quantizer.

Run where the reference's sources are available:

    python tests/golden/make_quant_golden.py <directory of the reference's sources>

The reference's ``binds/python/tests/test_nvfp4effma.py`` holds ``ref_quantize`` (Transformer Engine's NVFP4 arithmetic in
plain float32 torch ops, device-agnostic).  That module cannot be imported without the reference's compiled extension
and a GPU, so this script parses the file, takes only the definitions it needs (``GRID``, ``FLT_MAX``, ``e2m1_rne``,
``e4m3_rn``, ``ref_quantize``) and executes them on the CPU; nothing of it is copied into this repository.  The fixture
holds seeded inputs with zero blocks, an underflowing block and a zero row (as the reference's own pytest case builds
them, test_nvfp4effma.py:171-174) and, per recipe, the packed nibbles, the E4M3 scale codes and the global the reference
function returns.  tests/test_oracle_quant.py compares the CPU oracle with it bit for bit.
"""
import ast
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_quant_golden.py <directory of the reference's sources>")
REF = sys.argv[1]
SRC = os.path.join(REF, "binds/python/tests/test_nvfp4effma.py")
WANT = {"GRID", "FLT_MAX", "e2m1_rne", "e4m3_rn", "ref_quantize"}

RECIPES = [  # (name, tile, fos, smax, row_scaled) -- the recipe matrix of test_nvfp4effma.py:149-159
    ("te_1x16", 1, 0, 448, False),
    ("te_16x16", 16, 0, 448, False),
    ("fos_mae_256", 1, 1, 256, False),
    ("fos_mse_16x16_256", 16, 2, 256, False),
    ("fos_mae_448", 1, 1, 448, False),
    ("row_scaled", 1, 0, 448, True),
    ("row_scaled_fos_mse", 1, 2, 256, True),
    ("fos_mae_16x16_256", 16, 1, 256, False),
]


def load_reference_functions():
    tree = ast.parse(open(SRC).read())
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANT:
            keep.append(node)
        elif isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id in WANT for t in node.targets):
            keep.append(node)
    ns = {"torch": torch, "DEV": "cpu"}
    exec(compile(ast.Module(body=keep, type_ignores=[]), SRC, "exec"), ns)
    return ns


def make_input(dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn((67, 320), generator=g) * 3.0).to(dtype)
    x[3, :16] = 0          # zero block
    x[5, 16:32] *= 1e-30   # block scale underflows to 0
    x[7] = 0               # zero row
    x[11, 32:48] *= 2e4    # a block whose scale saturates
    return x


def main():
    ns = load_reference_functions()
    out = {}
    for dname, dtype in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        x = make_input(dtype, 1234)
        out[f"x_{dname}"] = x.float().numpy()
        for name, tile, fos, smax, row_scaled in RECIPES:
            data, code, gv = ns["ref_quantize"](x, tile=tile, fos=fos, smax=smax, row_scaled=row_scaled)
            out[f"{dname}/{name}/data"] = data.numpy().astype(np.uint8)
            out[f"{dname}/{name}/scales"] = code.view(torch.uint8).numpy()
            out[f"{dname}/{name}/global"] = gv.reshape(-1).float().numpy()
        # a given decode factor (ModelOpt form) instead of the amax
        g = torch.tensor([0.0625], dtype=torch.float32)
        data, code, gv = ns["ref_quantize"](x, g=g, tile=1, fos=0, smax=448)
        out[f"{dname}/given_g/data"] = data.numpy().astype(np.uint8)
        out[f"{dname}/given_g/scales"] = code.view(torch.uint8).numpy()
        out[f"{dname}/given_g/global"] = gv.reshape(-1).float().numpy()
    out["recipes"] = np.array([f"{n}:{t}:{f}:{s}:{int(r)}" for n, t, f, s, r in RECIPES])
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_torch_ref.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
