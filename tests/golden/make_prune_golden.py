"""Generate tests/golden/prune_masks.npz by running the reference's own gen_prune_mask.

The function is taken as text from ResNet-18-var/prune_script.py (the module itself imports TensorFlow
and cannot be imported here), executed on seeded inputs, and its masks and pruned arrays stored.

    python tests/golden/make_prune_golden.py <reference checkout>
"""
import ast
import os
import sys

import numpy as np

if len(sys.argv) < 2 and not os.environ.get("WG_REF"):
    sys.exit("usage: python tests/golden/make_prune_golden.py <reference checkout>   (or WG_REF=<checkout>)")
ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["WG_REF"]
src = open(os.path.join(ref, "ResNet-18-var", "prune_script.py")).read().replace("\t", "    ")
tree = ast.parse("\n".join(l for l in src.splitlines() if not l.strip().startswith("print ")))
fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "gen_prune_mask")
ns = {"np": np}
exec(compile(ast.Module(body=[fn], type_ignores=[]), "prune_script.py", "exec"), ns)
gen = ns["gen_prune_mask"]

rng = np.random.default_rng(2018)
blob = {}
for i, (shape, density) in enumerate([((16, 8, 12), 0.5), ((16, 32, 32), 0.3), ((16, 5, 7), 0.12), ((16, 4, 4), 0.0),
                                      ((16, 6, 10), 1.0), ((16, 16, 24), 0.35)]):
    w = rng.standard_normal(shape).astype(np.float32)
    blob["w%d" % i] = w.copy()
    blob["density%d" % i] = np.float64(density)
    pruned = w.copy()
    blob["mask%d" % i] = gen(pruned, density)
    blob["pruned%d" % i] = pruned
    # second round on the already masked weight, as the iterative ladder does (prune_script.py:71-72)
    again = (w * blob["mask%d" % i]).astype(np.float32)
    blob["mask2_%d" % i] = gen(again, density * 0.5)
out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "prune_masks.npz")
np.savez_compressed(out, **blob)
print("wrote", out)
