"""Generates level_draws.json by running the reference's own level-draw code.

The function body of CuHNSW.set_random_levels is taken from the reference's
cuhnsw/pyhnsw.py with `ast` (the module itself cannot be imported: it needs the
compiled binding) and executed unchanged against a stand-in `self`.  Run from
the repository root:   python tests/golden/make_level_draws.py /path/to/reference
"""
import ast
import hashlib
import json
import math
import os
import sys

import numpy as np

CASES = [  # (num_data, seed, level_mult expression)
  (1000, 777, 1 / math.log(12)),
  (100_000, 777, 1 / math.log(24)),
  (100_000, 777, 1 / math.log(12)),
  (1_183_514, 777, 1 / math.log(24)),
  (1_000_000, 777, 1 / math.log(32)),
  (12_500_000, 777, 1 / math.log(32)),
  (50_000, 42, 1 / math.log(16)),
]


def reference_function(ref_root):
  src = open(os.path.join(ref_root, "cuhnsw", "pyhnsw.py")).read()
  tree = ast.parse(src)
  consts = [n for n in tree.body if isinstance(n, ast.Assign) and getattr(n.targets[0], "id", "") == "EPS"]
  cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "CuHNSW")
  fn = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == "set_random_levels")
  ns = {"np": np}
  exec(compile(ast.Module(body=consts + [fn], type_ignores=[]), "pyhnsw.py", "exec"), ns)  # pylint: disable=exec-used
  return ns["set_random_levels"]


class _Obj:
  def set_random_levels(self, levels):
    self.levels = np.array(levels, copy=True)


class _Self:
  def __init__(self, n, seed, mult):
    self.opt = type("Opt", (), {"seed": seed, "level_mult": mult})()
    self.data = np.empty((n, 1), np.float32)
    self.obj = _Obj()


def main():
  ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
  if not ref_root:
    raise SystemExit("usage: make_level_draws.py <path of the reference checkout>  (or set REFERENCE_ROOT)")
  fn = reference_function(ref_root)
  out = []
  for n, seed, mult in CASES:
    me = _Self(n, seed, mult)
    fn(me)
    lv = me.obj.levels
    assert lv.dtype == np.int32
    mx = int(lv.max())
    out.append({
      "num_data": n, "seed": seed, "level_mult": mult, "max_level": mx,
      # first node reaching the maximum level (cpp/src/cuhnsw_base.cu:134-141)
      "enter_point": int(np.argmax(lv == mx)),
      "nodes_per_level": [int((lv >= l).sum()) for l in range(mx + 1)],
      "first_64": [int(x) for x in lv[:64]],
      "sha256": hashlib.sha256(lv.tobytes()).hexdigest(),
    })
  path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "level_draws.json")
  with open(path, "w") as f:
    json.dump(out, f, indent=1)
  print("wrote", path)


if __name__ == "__main__":
  main()
