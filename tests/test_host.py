"""Host-side logic that runs without a GPU: the C ABI surface, option handling, error
behaviour of the binding, benchmark arithmetic."""
import ctypes
import json
import math
import os
import re
import tempfile

import numpy as np
import pytest

from conftest import ROOT, has_gpu
from cuhnsw_b200 import aux
from cuhnsw_b200 import cuhnsw_bind
from cuhnsw_b200.cuhnsw_bind import CuHNSWBind


def declared_functions():
  text = open(os.path.join(ROOT, "include", "cuhnsw_b200.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  return sorted(set(re.findall(r"\b(cuhnsw_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
  names = declared_functions()
  assert len(names) >= 18
  lib = ctypes.CDLL(cuhnsw_bind.LIB_PATH)
  for name in names:
    assert hasattr(lib, name), f"{name} is declared in include/cuhnsw_b200.h but not exported"
  assert set(names) == set(cuhnsw_bind.SIGNATURES), "binding table and header disagree"


def test_create_destroy_and_null_handle():
  lib = cuhnsw_bind.load_library()
  h = lib.cuhnsw_create()
  assert h
  assert lib.cuhnsw_last_error(h) == b""
  lib.cuhnsw_destroy(h)
  assert lib.cuhnsw_init(None, b"x") == -1
  assert lib.cuhnsw_last_error(None) == b"null handle"
  assert lib.cuhnsw_merge_topk_device(None, None, 0, 0, 10, None, None, None, None) == -1


def write_opt(tmp, content):
  p = os.path.join(tmp, "opt.json")
  with open(p, "w") as f:
    f.write(content if isinstance(content, str) else json.dumps(content))
  return p


def test_init_error_behaviour_matches_reference_binding():
  """init() returns False for an unreadable or malformed option file (cuhnsw_base.cu:69,75)
  and raises for an invalid distance type (cuhnsw_base.cu:95-101)."""
  with tempfile.TemporaryDirectory() as tmp:
    b = CuHNSWBind()
    assert b.init(os.path.join(tmp, "missing.json")) is False
    assert b.init(write_opt(tmp, "{not json")) is False
    assert b.init(write_opt(tmp, '{"a": {"b": 1}}')) is False
    assert b.init(write_opt(tmp, '{"a": [1, [2]]}')) is False
    assert b.init(write_opt(tmp, '{"a": [1, "x"]}')) is False
    with pytest.raises(RuntimeError, match="invalid dist type hamming"):
      b.init(write_opt(tmp, {"dist_type": "hamming"}))
    with pytest.raises(RuntimeError, match="max_m"):
      b.init(write_opt(tmp, {"max_m": 40, "max_m0": 24}))
    with pytest.raises(RuntimeError, match="heuristic_coef"):
      b.init(write_opt(tmp, {"heuristic_coef": 1.5}))
    assert b.init(write_opt(tmp, {"reverse_cand": True})) is True
    assert b.init(write_opt(tmp, {"dist_type": "l2", "heuristic_coff": 0.5, "unknown_key": 3})) is True
    assert b.init(write_opt(tmp, "{}")) is True


def test_call_order_and_argument_checks():
  with tempfile.TemporaryDirectory() as tmp:
    b = CuHNSWBind()
    with pytest.raises(RuntimeError, match="init"):
      b.set_data(np.zeros((2, 4), np.float32))
    assert b.init(write_opt(tmp, {}))
    with pytest.raises(RuntimeError, match="2d"):
      b.set_data(np.zeros(4, np.float32))
    with pytest.raises(RuntimeError, match="1d"):
      b.set_random_levels(np.zeros((2, 2), np.int32))
    with pytest.raises(RuntimeError, match="set_data"):
      b.set_random_levels(np.zeros(2, np.int32))
    with pytest.raises(RuntimeError, match="set_random_levels"):
      b.build_graph()
    with pytest.raises(RuntimeError, match="no graph"):
      b.save_index(os.path.join(tmp, "x.index"))
    q, nns = np.zeros((1, 4), np.float32), np.zeros((1, 3), np.int32)
    with pytest.raises(RuntimeError, match="no graph"):
      b.search_knn(q, 3, 10, nns, np.zeros((1, 3), np.float32), np.zeros(1, np.int32))
    with pytest.raises(RuntimeError, match="float32"):
      b.search_knn(q, 3, 10, nns, np.zeros((1, 3), np.float64), np.zeros(1, np.int32))
    # both host-buffer searches check their output arrays before anything is written through them
    for search in (b.search_knn, b.search_knn_noalloc):
      with pytest.raises(RuntimeError, match="float32"):
        search(q, 3, 10, nns, np.zeros((1, 3), np.float64), np.zeros(1, np.int32))
      with pytest.raises(RuntimeError, match="too small"):
        search(q, 3, 10, np.zeros((1, 2), np.int32), np.zeros((1, 3), np.float32), np.zeros(1, np.int32))
      with pytest.raises(RuntimeError, match="int32"):
        search(q, 3, 10, nns, np.zeros((1, 3), np.float32), np.zeros(1, np.int64))
      with pytest.raises(RuntimeError, match="writable"):
        ro = np.zeros((1, 3), np.float32)
        ro.flags.writeable = False
        search(q, 3, 10, nns, ro, np.zeros(1, np.int32))
      with pytest.raises(RuntimeError, match="topk"):
        search(q, 0, 10, nns, np.zeros((1, 3), np.float32), np.zeros(1, np.int32))
    # the asynchronous search takes raw addresses; without a graph it must refuse before touching them
    with pytest.raises(RuntimeError, match="no graph"):
      b.search_knn_async(q.ctypes.data, 1, 3, 10, nns.ctypes.data, 0, 0)
    with pytest.raises(RuntimeError, match="cannot open"):
      b.load_index(os.path.join(tmp, "nope.index"))
    short = os.path.join(tmp, "short.index")
    open(short, "wb").write(b"\0" * 40)
    with pytest.raises(RuntimeError, match="shorter than its header"):
      b.load_index(short)
    bad = os.path.join(tmp, "bad.index")
    open(bad, "wb").write(b"\xff" * 200)
    with pytest.raises(RuntimeError, match="index file"):
      b.load_index(bad)


@pytest.mark.skipif(has_gpu(), reason="checks the failure mode of a machine without a GPU")
def test_fails_loudly_without_a_gpu():
  with tempfile.TemporaryDirectory() as tmp:
    b = CuHNSWBind()
    assert b.init(write_opt(tmp, {}))
    with pytest.raises(RuntimeError, match="no CUDA device"):
      b.set_data(np.zeros((4, 8), np.float32))
    # the helpers of the asynchronous search fail the same way instead of handing out null streams or buffers
    with pytest.raises(RuntimeError, match="no CUDA device"):
      b.stream_create()
    with pytest.raises(RuntimeError, match="page-lock"):
      b.host_array((4, 8), np.float32)


def test_option_schema_matches_config_proto():
  expected = dict(seed=777, c_log_level=2, py_log_level=2, max_m=12, max_m0=24, ef_construction=150, level_mult=0.0,
                  save_remains=False, hyper_threads=10.0, block_dim=32, dist_type="dot", visited_table_size=0,
                  visited_list_size=8192, nrz=False, reverse_cand=False, heuristic_coef=0.25)
  proto = aux.get_opt_as_proto({})
  for key, val in expected.items():
    assert getattr(proto, key) == val and type(getattr(proto, key)) is type(val), key
  assert set(aux.SCHEMA) == set(expected)
  with pytest.raises(AttributeError):
    aux.get_opt_as_proto({"ef_search": 50})
  with pytest.raises(TypeError):
    aux.get_opt_as_proto({"max_m": "12"})
  with pytest.raises(TypeError):
    aux.get_opt_as_proto({"nrz": 1})
  assert aux.get_opt_as_proto({"heuristic_coff": 0.5}).heuristic_coef == 0.5
  assert aux.get_opt_as_proto({"hyper_threads": 100}).hyper_threads == 100.0
  d = aux.proto_to_dict(aux.get_opt_as_proto({"max_m": 16}))
  assert d["max_m"] == 16 and json.loads(json.dumps(d)) == d
  assert aux.load_json_string('{"a": 1, // c\n "b": [1, 2,],}') == {"a": 1, "b": [1, 2]}


def test_extension_options_and_their_validation():
  """Keys this engine adds to the reference's schema: defaults, types, and what the C++ side refuses."""
  proto = aux.get_opt_as_proto({})
  assert (proto.batch_max, proto.ramp_div, proto.device_id) == (0, 4, -1)
  assert (proto.search_team, proto.search_schedule, proto.row_dtype) == (-1, True, "f32")
  assert proto.devices == [] and aux.proto_to_dict(aux.get_opt_as_proto({"devices": [0, 1]}))["devices"] == [0, 1]
  with pytest.raises(TypeError):
    aux.get_opt_as_proto({"devices": "0,1"})
  d = aux.proto_to_dict(aux.get_opt_as_proto({"row_dtype": "f16", "search_schedule": False, "search_team": 1}))
  assert d["row_dtype"] == "f16" and d["search_schedule"] is False and d["search_team"] == 1
  with pytest.raises(TypeError):
    aux.get_opt_as_proto({"row_dtype": 16})
  with tempfile.TemporaryDirectory() as tmp:
    b = CuHNSWBind()
    assert b.init(write_opt(tmp, {"row_dtype": "f16", "search_schedule": False}))
    assert b.init(write_opt(tmp, {"devices": [0, 1, 1]}))
    assert b.init(write_opt(tmp, {"devices": []}))
    with pytest.raises(RuntimeError, match="devices"):
      b.init(write_opt(tmp, {"devices": [0, -1]}))
    with pytest.raises(RuntimeError, match="disagree"):
      b.init(write_opt(tmp, {"devices": [1, 0], "device_id": 0}))
    assert b.init(write_opt(tmp, {"row_dtype": "bf16"}))
    with pytest.raises(RuntimeError, match="row_dtype must be f32, f16 or bf16"):
      CuHNSWBind().init(write_opt(tmp, {"row_dtype": "f8"}))


def test_python_api_constructor_semantics():
  from cuhnsw_b200 import CuHNSW
  c = CuHNSW({"py_log_level": 1, "c_log_level": 0})
  assert c.opt.level_mult == pytest.approx(1 / math.log(12))  # cuhnsw/pyhnsw.py:26 uses max_m
  assert CuHNSW({"dist_type": "euclidean", "py_log_level": 1}).opt.dist_type == "l2"
  assert CuHNSW({"dist_type": "cosine", "py_log_level": 1}).opt.dist_type == "dot"
  assert CuHNSW({"dist_type": "ip", "py_log_level": 1}).opt.dist_type == "dot"
  with pytest.raises(AssertionError):
    CuHNSW({"dist_type": "hamming"})
  with pytest.raises(AssertionError):
    CuHNSW({"block_dim": 48})


def test_benchmark_arithmetic():
  import bench
  assert bench.algorithmic_bytes_per_query(10, 2, 1, 50, 12, 24, 10) == 10 * 200 + 2 * 100 + 52 + 200 + 80
  assert bench.algorithmic_bytes_per_query(10, 2, 1, 50, 12, 24, 10, 2) == 10 * 100 + 2 * 100 + 52 + 200 + 80
  assert bench.pick_ef({50: 0.9, 100: 0.96, 300: 0.99}) == 100
  assert bench.pick_ef({50: 0.5, 100: 0.6}) == 100
  peak, kind = bench.measured_peak()
  assert peak > 1000 and kind in ("measured", "fallback")
