"""One handle over several GPUs (option ``devices``): the index is built once and copied to every listed
GPU, and a host-buffer search is cut into contiguous slices, one per GPU.  The reference is single-device
(cpp/src/cuhnsw_build.cu:15-23 takes the current device).  A device may be listed twice, which gives two
replicas on one GPU: that exercises the whole split, copy and join logic on a single-GPU machine."""
import numpy as np
import pytest

from conftest import assert_same_bits, engine_options, has_gpu, small_workload
from cuhnsw_b200 import CuHNSW

pytestmark = pytest.mark.gpu


def gpu_count():
  if not has_gpu():
    return 0
  import torch
  return torch.cuda.device_count()


def device_lists():
  n = gpu_count()
  lists = [[0, 0], [0, 0, 0]]
  if n >= 2:
    lists += [[0, 1], list(range(n))]
  return lists


@pytest.mark.parametrize("devices", device_lists(), ids=str)
def test_search_split_over_replicas_equals_single_gpu_search(devices, tmp_path):
  base, q, opt = small_workload("angular_toy", 20000, 1003)
  one = CuHNSW(engine_options(opt))
  one.set_data(base)
  one.build()
  many = CuHNSW(engine_options(opt, devices=devices))
  many.set_data(base)
  many.build()
  for queries, topk, ef in ((q, 10, 100), (q[:1], 10, 50), (q[:2], 5, 20), (q[:len(devices) - 1], 3, 10)):
    want = one.search_knn(queries, topk, ef)
    got = many.search_knn(queries, topk, ef)
    assert (got[0] == want[0]).all() and (got[2] == want[2]).all()
    assert_same_bits(got[1], want[1])
  # a loaded (labelled) index is replicated with its labels; a new build replaces the replicas
  path = str(tmp_path / "m.index")
  one.save_index(path)
  many.load_index(path)
  got, want = many.search_knn(q, 10, 64), one.search_knn(q, 10, 64)
  assert (got[0] == want[0]).all()
  many.set_data(base[:5000])
  many.build()
  one.set_data(base[:5000])
  one.build()
  got, want = many.search_knn(q, 10, 64), one.search_knn(q, 10, 64)
  assert (got[0] == want[0]).all()
  assert_same_bits(got[1], want[1])


def test_a_device_that_does_not_exist_is_an_error_not_a_hang():
  base, q, opt = small_workload("angular_toy", 2000, 16)
  eng = CuHNSW(engine_options(opt, devices=[0, 999], c_log_level=0))
  eng.set_data(base)
  with pytest.raises(RuntimeError, match="device 999"):
    eng.build()  # the copy to the second GPU fails; the message names it
  with pytest.raises(RuntimeError, match="device 999"):
    eng.search_knn(q, 10, 20)
  # the same data on the GPUs that exist still works
  ok = CuHNSW(engine_options(opt, devices=[0]))
  ok.set_data(base)
  ok.build()
  assert (ok.search_knn(q, 10, 20)[2] == 10).all()


@pytest.mark.parametrize("devices", device_lists(), ids=str)
def test_batches_in_flight_go_round_the_replicas(devices):
  """CuHNSW.search_knn_batches on a handle with `devices`: consecutive batches go to consecutive replicas
  (cuhnsw_search_knn_async_on), several per replica in flight; answers equal the single-GPU answers and come
  back in order; the caller's current device is what it was."""
  import torch
  base, q, opt = small_workload("angular_toy", 20000, 3000)
  one = CuHNSW(engine_options(opt))
  one.set_data(base)
  one.build()
  many = CuHNSW(engine_options(opt, devices=devices))
  many.set_data(base)
  many.build()
  assert many.obj.replica_count() == len(devices) and one.obj.replica_count() == 1
  batches = [np.roll(q, 211 * i, axis=0)[:m] for i, m in enumerate([3000, 5, 1500, 3000, 1, 2999, 64, 800, 3000])]
  before = torch.cuda.current_device()
  got = list(many.search_knn_batches(batches, 10, 64, in_flight=2))
  assert torch.cuda.current_device() == before
  assert len(got) == len(batches)
  for b, (ids, dist, found) in zip(batches, got):
    want = one.search_knn(b, 10, 64)
    assert (ids == want[0]).all() and (found == want[2]).all()
    assert_same_bits(dist, want[1])
  # a rebuild on the primary reaches the replicas before the next batch does
  many.set_data(base[:4000])
  many.build()
  one.set_data(base[:4000])
  one.build()
  got = list(many.search_knn_batches(batches[:4], 10, 64, in_flight=1))
  for b, (ids, dist, found) in zip(batches[:4], got):
    assert (ids == one.search_knn(b, 10, 64)[0]).all()
  with pytest.raises(RuntimeError, match="no replica"):
    many.obj.stream_create(len(devices))
