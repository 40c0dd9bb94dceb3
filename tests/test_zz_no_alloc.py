"""The search entry point for callers that cannot allocate device memory.

Some users of this library run inside a process whose GPU memory is already spoken for: a
serving framework that grabbed all free memory for its own pool, a job with a hard memory
budget, or a loop that cannot afford the device-wide synchronisation an allocation brings.
For them `cuhnsw_search_knn_noalloc` keeps its device staging in a fixed 4 MiB array inside
the library.  This file checks, through the C ABI, that it returns exactly what
`cuhnsw_search_knn` returns (ids and counts equal, distances bit-equal: the tolerance the
other parity tests use), on two calls in a row that share the array, and that a request
beyond the array's size is refused with a clear message.  It is collected last on purpose.
"""
import numpy as np
import pytest

from conftest import assert_same_bits, engine_options, small_workload
from cuhnsw_b200 import CuHNSW

pytestmark = pytest.mark.gpu


def outputs(nq, topk):
  return (np.full((nq, topk), -7, np.int32), np.full((nq, topk), -7.0, np.float32), np.full((nq,), -7, np.int32))


def test_noalloc_search_equals_regular_search_on_consecutive_calls():
  base, q, opt = small_workload("angular_toy", 20000, 900)
  eng = CuHNSW(engine_options(opt, batch_max=1024))
  eng.set_data(base)
  eng.build()
  # two back-to-back calls with different shapes: the second is smaller, uses another ef and topk, so
  # anything left over from the first call in the shared array would show up as a difference
  for queries, topk, ef in ((q[:900], 10, 120), (q[100:350], 7, 40)):
    want = outputs(len(queries), topk)
    eng.obj.search_knn(queries, topk, ef, *want)
    got = outputs(len(queries), topk)
    eng.obj.search_knn_noalloc(queries, topk, ef, *got)
    assert (got[0] == want[0]).all()
    assert (got[2] == want[2]).all() and (got[2] == topk).all()
    assert_same_bits(got[1], want[1])
  # a second handle in the same process shares the same array
  other = CuHNSW(engine_options(opt, batch_max=1024))
  other.set_data(base[:5000])
  other.build()
  want, got = outputs(64, 10), outputs(64, 10)
  other.obj.search_knn(q[:64], 10, 50, *want)
  other.obj.search_knn_noalloc(q[:64], 10, 50, *got)
  assert (got[0] == want[0]).all() and (got[2] == want[2]).all()
  assert_same_bits(got[1], want[1])


def test_noalloc_search_rejects_requests_beyond_its_fixed_array():
  base, q, opt = small_workload("angular_toy", 2000, 16)
  eng = CuHNSW(engine_options(opt, batch_max=256))
  eng.set_data(base)
  eng.build()
  nq = 30000  # 30000 x 50 floats alone are 6 MB > 4 MiB
  big = np.zeros((nq, 50), np.float32)
  with pytest.raises(RuntimeError, match=r"limit is 4194304"):
    eng.obj.search_knn_noalloc(big, 10, 20, *outputs(nq, 10))
  # the handle stays usable, and the largest documented batch fits
  fit = np.tile(q, (625, 1))[:10000]
  got, want = outputs(10000, 10), outputs(10000, 10)
  eng.obj.search_knn_noalloc(fit, 10, 20, *got)
  eng.obj.search_knn(fit, 10, 20, *want)
  assert (got[0] == want[0]).all() and (got[2] == want[2]).all()
  assert_same_bits(got[1], want[1])


@pytest.mark.parametrize("d,row_dtype,nq,labelled", [(50, "f32", 300, False), (200, "f32", 40, False), (200, "f32", 2000, True),
                                                     (96, "f16", 300, True), (50, "bf16", 300, False)])
def test_noalloc_search_takes_no_device_memory_once_warm(d, row_dtype, nq, labelled, tmp_path):
  """The promise is about device memory: after one warm-up call (which loads the search kernel of this row
  width, row type and batch class, and looks the fixed array up), a call must leave the amount of free device
  memory exactly where it was.  Covers rows wider than 128 floats (the CTA-per-query kernel for few queries, the
  warp-per-query kernel for many), 16-bit rows and an index that came from a file (ids mapped through labels)."""
  import torch
  rng = np.random.default_rng(d + nq)
  n = 6000
  base = rng.standard_normal((n, d)).astype(np.float32)
  q = rng.standard_normal((nq, d)).astype(np.float32)
  opt = {"dist_type": "l2", "max_m": 12, "max_m0": 24, "ef_construction": 60, "seed": 3, "row_dtype": row_dtype,
         "batch_max": 500}
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  if labelled:
    path = str(tmp_path / "n.index")
    eng.save_index(path)
    eng = CuHNSW(engine_options({"dist_type": "l2", "row_dtype": row_dtype}))
    eng.load_index(path)
  want, got = outputs(nq, 10), outputs(nq, 10)
  eng.obj.search_knn(q, 10, 80, *want)
  eng.obj.search_knn_noalloc(q, 10, 80, *got)  # warm-up: kernel load + address look-up
  torch.cuda.synchronize()
  free_before = torch.cuda.mem_get_info()[0]
  for _ in range(3):
    got = outputs(nq, 10)
    eng.obj.search_knn_noalloc(q, 10, 80, *got)
  torch.cuda.synchronize()
  assert torch.cuda.mem_get_info()[0] == free_before, "a warmed-up call changed the free device memory"
  assert (got[0] == want[0]).all() and (got[2] == want[2]).all()
  assert_same_bits(got[1], want[1])
