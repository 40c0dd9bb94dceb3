"""hnswlib-compatible index file, restated with numpy for the tests.

TEST INFRASTRUCTURE ONLY.  An independent reader/writer of the byte layout the
reference writes in cpp/src/cuhnsw_base.cu:159-247 and reads back in
cpp/src/cuhnsw_base.cu:250-365, used to check the library's own C++ file code:

  header (96 B, little endian):
    u64 offsetLevel0 (=0), u64 max_elements, u64 cur_element_count,
    u64 size_data_per_element, u64 label_offset, u64 offsetData,
    i32 maxlevel, u32 enterpoint_node, u64 maxM, u64 maxM0, u64 M,
    f64 mult, u64 ef_construction
  cur_element_count level-0 records of size_data_per_element bytes:
    u32 degree | maxM0 x u32 ids | d x f32 | u64 label
  then, per node: u32 nbytes = levels[i] * (4 + 4*maxM), followed by
    levels[i] records  u32 degree | maxM x u32 ids   (levels 1..levels[i])
"""
import struct

import numpy as np

from . import Graph

HEADER = struct.Struct("<QQQQQQiIQQQdQ")
assert HEADER.size == 96


def read_header(buf):
  (off0, max_elements, count, size_per_elem, label_offset, offset_data, maxlevel, enter, max_m, max_m0, m,
   mult, efc) = HEADER.unpack_from(buf, 0)
  return dict(offsetLevel0=off0, max_elements=max_elements, cur_element_count=count,
              size_data_per_element=size_per_elem, label_offset=label_offset, offsetData=offset_data,
              maxlevel=maxlevel, enterpoint_node=enter, maxM=max_m, maxM0=max_m0, M=m, mult=mult,
              ef_construction=efc)


def load(path, dist_type):
  with open(path, "rb") as f:
    buf = f.read()
  h = read_header(buf)
  n, max_m, max_m0 = h["cur_element_count"], h["maxM"], h["maxM0"]
  d = (h["label_offset"] - h["offsetData"]) // 4
  rec = h["size_data_per_element"]
  assert rec == 4 + 4 * max_m0 + 4 * d + 8
  body = np.frombuffer(buf, np.uint8, n * rec, HEADER.size).reshape(n, rec)
  deg0 = body[:, 0:4].copy().view(np.uint32).reshape(n) & 0xffff
  rows0 = body[:, 4:4 + 4 * max_m0].copy().view(np.uint32).reshape(n, max_m0).astype(np.int32)
  vec = body[:, 4 + 4 * max_m0:4 + 4 * max_m0 + 4 * d].copy().view(np.float32).reshape(n, d)
  labels = body[:, rec - 8:].copy().view(np.uint64).reshape(n)
  pos = HEADER.size + n * rec
  per_link = 4 + 4 * max_m
  levels = np.zeros(n, np.int32)
  upper = []
  for i in range(n):
    (nbytes,) = struct.unpack_from("<I", buf, pos)
    pos += 4
    levels[i] = nbytes // per_link
    if nbytes:
      upper.append(np.frombuffer(buf, np.uint32, nbytes // 4, pos).reshape(levels[i], 1 + max_m))
      pos += nbytes
  assert pos == len(buf), (pos, len(buf))
  g = Graph(vec, levels, max_m, max_m0, dist_type)
  g.deg0[:] = deg0.astype(np.int32)
  g.rows0[:] = rows0
  g.rows0[np.arange(max_m0)[None, :] >= g.deg0[:, None]] = -1
  if upper:
    allu = np.concatenate(upper, axis=0)
    g.degU[:allu.shape[0]] = (allu[:, 0] & 0xffff).astype(np.int32)
    g.rowsU[:allu.shape[0]] = allu[:, 1:].astype(np.int32)
    g.rowsU[np.arange(max_m)[None, :] >= g.degU[:, None]] = -1
  g.max_level = h["maxlevel"]
  g.enter_point = h["enterpoint_node"]
  g.labels = labels.astype(np.int64)
  g.header = h
  return g


def save(path, g, level_mult, ef_construction, labels=None):
  n, d, max_m, max_m0 = g.n, g.d, g.max_m, g.max_m0
  rec = 4 + 4 * max_m0 + 4 * d + 8
  out = bytearray(HEADER.pack(0, n, n, rec, 4 + 4 * max_m0 + 4 * d, 4 + 4 * max_m0, g.max_level,
                              g.enter_point, max_m, max_m0, max_m, float(level_mult), ef_construction))
  body = np.zeros((n, rec), np.uint8)
  body[:, 0:4] = g.deg0.astype(np.uint32).view(np.uint8).reshape(n, 4)
  rows = np.where(g.rows0 >= 0, g.rows0, 0).astype(np.uint32)
  body[:, 4:4 + 4 * max_m0] = rows.view(np.uint8).reshape(n, 4 * max_m0)
  body[:, 4 + 4 * max_m0:4 + 4 * max_m0 + 4 * d] = g.vec.view(np.uint8).reshape(n, 4 * d)
  lab = (np.arange(n) if labels is None else np.asarray(labels)).astype(np.uint64)
  body[:, rec - 8:] = lab.view(np.uint8).reshape(n, 8)
  out += body.tobytes()
  for i in range(n):
    lv = int(g.levels[i])
    out += struct.pack("<I", lv * (4 + 4 * max_m))
    for l in range(lv):
      r = int(g.upper_base[i]) + l
      out += struct.pack("<I", int(g.degU[r]))
      out += np.where(g.rowsU[r] >= 0, g.rowsU[r], 0).astype(np.uint32).tobytes()
  with open(path, "wb") as f:
    f.write(bytes(out))
