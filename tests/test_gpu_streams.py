"""Searches enqueued on different streams may run at the same time: every stream has its own ticket counter,
schedule arrays and staging buffers inside the engine.  The reference's SearchGraph blocks and has one set of
buffers per call (cpp/src/cuhnsw_build.cu:210-290), so there is nothing to compare with but this engine's own
blocking search, which in turn is tested against the oracle."""
import numpy as np
import pytest

from conftest import assert_same_bits, engine_options, small_workload
from cuhnsw_b200 import CuHNSW

pytestmark = pytest.mark.gpu


def _engine(n, nq, **extra):
  base, q, opt = small_workload("angular_toy", n, nq)
  eng = CuHNSW(engine_options(opt, **extra))
  eng.set_data(base)
  eng.build()
  return eng, q


@pytest.mark.parametrize("streams", [2, 3, 10])
def test_device_searches_on_several_streams_give_the_blocking_answers(streams):
  """7000 queries per batch: more than one wave, so every batch also uses its stream's schedule arrays.  Ten
  streams are more than the engine keeps scratch for: the ninth and tenth take over a set after a wait."""
  import torch
  eng, q = _engine(30000, 7000)
  batches = [np.ascontiguousarray(np.roll(q, 911 * b, axis=0)) for b in range(12)]
  want = [eng.search_knn(b, 10, 48) for b in batches]
  pool = [torch.cuda.Stream() for _ in range(streams)]
  dq = [torch.from_numpy(b).cuda() for b in batches]
  out = [(torch.full((len(q), 10), -7, dtype=torch.int32, device="cuda"), torch.zeros((len(q), 10), device="cuda"),
          torch.zeros(len(q), dtype=torch.int32, device="cuda")) for _ in batches]
  torch.cuda.synchronize()
  for rounds in range(2):
    for b in range(len(batches)):
      eng.obj.set_stream(pool[b % streams].cuda_stream)
      eng.obj.search_knn_device(dq[b].data_ptr(), len(q), 10, 48, out[b][0].data_ptr(), out[b][1].data_ptr(),
                                out[b][2].data_ptr())
  torch.cuda.synchronize()
  eng.obj.set_stream(0)
  for b in range(len(batches)):
    assert (out[b][0].cpu().numpy() == want[b][0]).all(), b
    assert (out[b][2].cpu().numpy() == want[b][2]).all(), b
    assert_same_bits(out[b][1].cpu().numpy(), want[b][1])


@pytest.mark.parametrize("zero_copy", [True, False])
def test_host_buffer_searches_without_the_wait_give_the_blocking_answers(zero_copy):
  """cuhnsw_search_knn_async with page-locked buffers on two streams, batches of different sizes.  With
  zero_copy (the default) the kernels read and write the page-locked buffers in place; without it they go
  through the stream's staging buffers, which grow between calls.  The expected answers come from pageable
  numpy arrays, which always take the staged path."""
  import torch
  eng, q = _engine(20000, 6000, zero_copy=zero_copy)
  sizes = [6000, 1, 2500, 6000, 37, 5999]
  batches = [np.ascontiguousarray(np.roll(q, 517 * i, axis=0)[:m]) for i, m in enumerate(sizes)]
  want = [eng.search_knn(b, 7, 40) for b in batches]
  pool = [torch.cuda.Stream() for _ in range(2)]
  hq = [torch.from_numpy(b).pin_memory() for b in batches]
  out = [(torch.full((m, 7), -7, dtype=torch.int32).pin_memory(), torch.zeros((m, 7)).pin_memory(),
          torch.zeros(m, dtype=torch.int32).pin_memory()) for m in sizes]
  for i, m in enumerate(sizes):
    eng.obj.set_stream(pool[i % 2].cuda_stream)
    eng.obj.search_knn_async(hq[i].data_ptr(), m, 7, 40, out[i][0].data_ptr(), out[i][1].data_ptr(),
                             out[i][2].data_ptr())
  for s in pool:
    s.synchronize()
  eng.obj.set_stream(0)
  for i in range(len(sizes)):
    assert (out[i][0].numpy() == want[i][0]).all(), i
    assert (out[i][2].numpy() == want[i][2]).all(), i
    assert_same_bits(out[i][1].numpy(), want[i][1])
  # the blocking call still works on the stream the asynchronous ones used, and on the default stream
  eng.obj.set_stream(pool[0].cuda_stream)
  again = eng.search_knn(batches[0], 7, 40)
  eng.obj.set_stream(0)
  assert (again[0] == want[0][0]).all()


def test_a_rebuild_waits_for_searches_in_flight_and_a_destroyed_stream_does_no_harm():
  """set_data / build / load_index replace what running searches read, so they first wait for every search
  enqueued so far, whatever its stream; a scratch set whose stream the caller has destroyed is reused through
  the set's own event, not through the stream."""
  import torch
  eng, q = _engine(20000, 7000)
  want = eng.search_knn(q, 10, 64)
  dq = torch.from_numpy(q).cuda()
  out = (torch.empty((len(q), 10), dtype=torch.int32, device="cuda"), torch.empty((len(q), 10), device="cuda"),
         torch.empty(len(q), dtype=torch.int32, device="cuda"))
  for turn in range(12):  # more short-lived streams than the engine has scratch sets
    side = torch.cuda.Stream()
    eng.obj.set_stream(side.cuda_stream)
    eng.obj.search_knn_device(dq.data_ptr(), len(q), 10, 64, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr())
    side.synchronize()
    assert (out[0].cpu().numpy() == want[0]).all(), turn
    eng.obj.set_stream(0)
    del side
  side = torch.cuda.Stream()
  eng.obj.set_stream(side.cuda_stream)
  eng.obj.search_knn_device(dq.data_ptr(), len(q), 10, 64, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr())
  eng.obj.set_stream(0)
  base, _, _ = small_workload("angular_toy", 5000, 16)
  eng.set_data(base)  # must not pull the rows from under the search above
  eng.build()
  torch.cuda.synchronize()
  assert (out[0].cpu().numpy() == want[0]).all()
  assert int(eng.search_knn(q[:100], 10, 64)[0].max()) < 5000


@pytest.mark.parametrize("in_flight", [1, 3])
def test_python_batch_generator_gives_the_blocking_answers_in_order(in_flight):
  """CuHNSW.search_knn_batches: batches of different sizes (a single 1-d query and an empty batch among them)
  through the library's own streams and page-locked buffers; also when the consumer stops early."""
  eng, q = _engine(20000, 6000)
  sizes = [6000, 1, 0, 2500, 6000, 37, 5999, 12]
  batches = [np.roll(q, 313 * i, axis=0)[:m] for i, m in enumerate(sizes)]
  batches[1] = batches[1][0]  # one query as a vector
  got = list(eng.search_knn_batches(iter(batches), 7, 40, in_flight=in_flight))
  assert len(got) == len(batches)
  for b, (ids, dist, found) in zip(batches, got):
    want = eng.search_knn(b, 7, 40) if len(np.atleast_2d(b)) and b.size else None
    if want is None:
      assert ids.shape == (0, 7) and dist.shape == (0, 7) and found.shape == (0,)
      continue
    assert (ids == want[0]).all() and (found == want[2]).all()
    assert_same_bits(dist, want[1])
  gen = eng.search_knn_batches(iter(batches), 7, 40, in_flight=in_flight)
  first = next(gen)
  gen.close()  # streams and buffers are released with searches still in flight
  assert (first[0] == eng.search_knn(batches[0], 7, 40)[0]).all()
  with pytest.raises(RuntimeError):
    list(eng.search_knn_batches([q[:, :10]], 7, 40))
