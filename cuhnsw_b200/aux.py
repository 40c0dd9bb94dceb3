"""Option handling and logging of the Python layer.

Same functions as cuhnsw/aux.py of js1010/cuhnsw (get_logger :18-36, Option :79-119,
get_opt_as_proto :60-67, proto_to_dict :69-72 there; Apache-2.0, Copyright (c) 2020 Jisang Yoon),
written anew.  The reference validates the
option dict by parsing it into a protobuf message generated from
cuhnsw/proto/config.proto; the generated module needs protoc, so the schema is
restated here as a typed table with the same field names, types and defaults,
and the same behaviour: unknown keys and wrongly typed values are rejected.
"""
import json
import logging
import re


_LEVELS = {1: logging.WARNING, 2: logging.INFO, 3: logging.DEBUG}
_LOG_FORMAT = "[%(levelname)-8s] %(asctime)s [%(filename)s] [%(funcName)s:%(lineno)d]%(message)s"


def get_logger(name=__file__, level=2):
  """Logger that writes to stderr.  ``level`` follows the option ``py_log_level``: 1 = warnings,
  2 = info, 3 = debug (the numbering of the reference's aux.get_logger); other values are passed to
  ``logging`` as they are.  A logger that already has a handler is returned unchanged."""
  logger = logging.getLogger(name)
  if not logger.handlers:
    threshold = _LEVELS.get(level, level)
    handler = logging.StreamHandler()
    handler.setLevel(threshold)
    handler.setFormatter(logging.Formatter(_LOG_FORMAT, "%Y-%m-%d %H:%M:%S"))
    logger.setLevel(threshold)
    logger.addHandler(handler)
  return logger


def load_json_string(cont):
  """JSON with // comments and trailing commas (aux.py:41-50 of the reference)."""
  cont = re.sub(r"(^|\s)//[^\n]*", r"\1", cont)
  cont = re.sub(",[ \t\r\n]*}", "}", cont)
  cont = re.sub(",[ \t\r\n]*" + r"\]", "]", cont)
  return json.loads(cont)


def load_json_file(fname):
  with open(fname, "r") as fin:
    return load_json_string(fin.read())


# field -> (type, default); None default = "not set" (proto2 optional without default)
SCHEMA = {
  "seed": (int, 777),
  "c_log_level": (int, 2),
  "py_log_level": (int, 2),
  "max_m": (int, 12),
  "max_m0": (int, 24),
  "ef_construction": (int, 150),
  "level_mult": (float, 0.0),
  "save_remains": (bool, False),
  "hyper_threads": (float, 10.0),
  "block_dim": (int, 32),
  "dist_type": (str, "dot"),
  "visited_table_size": (int, 0),
  "visited_list_size": (int, 8192),
  "nrz": (bool, False),
  "reverse_cand": (bool, False),
  "heuristic_coef": (float, 0.25),
}
# keys this engine adds; optional, never required
EXTENSIONS = {
  "batch_max": (int, 0),
  "ramp_div": (int, 4),
  "device_id": (int, -1),
  "search_team": (int, -1),
  "search_schedule": (bool, True),
  "zero_copy": (bool, True),
  "row_dtype": (str, "f32"),
  # GPUs that hold a replica of the index and share every host-buffer search; empty = one GPU (device_id)
  "devices": (list, ()),
}
ALIASES = {"heuristic_coff": "heuristic_coef"}


class ConfigProto:
  """Attribute bag with the fields of the reference's ConfigProto message."""

  def __init__(self):
    for key, (typ, default) in {**SCHEMA, **EXTENSIONS}.items():
      object.__setattr__(self, key, list(default) if typ is list else default)

  def __setattr__(self, key, value):
    table = {**SCHEMA, **EXTENSIONS}
    if key not in table:
      raise AttributeError(f"ConfigProto has no field {key}")
    object.__setattr__(self, key, _coerce(key, table[key][0], value))

  def IsInitialized(self, errors=None):  # proto2 API used by the reference; no required fields exist
    return True


def _coerce(key, typ, value):
  if typ is bool:
    if isinstance(value, bool):
      return value
    raise TypeError(f"option {key}: expected bool, got {value!r}")
  if typ is int:
    if isinstance(value, bool) or not isinstance(value, (int,)) and not (
        isinstance(value, float) and float(value).is_integer()):
      raise TypeError(f"option {key}: expected int, got {value!r}")
    return int(value)
  if typ is list:
    if isinstance(value, (str, bytes)) or not all(isinstance(v, int) and not isinstance(v, bool) for v in value):
      raise TypeError(f"option {key}: expected a list of ints, got {value!r}")
    return [int(v) for v in value]
  if typ is float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
      raise TypeError(f"option {key}: expected number, got {value!r}")
    return float(value)
  if not isinstance(value, str):
    raise TypeError(f"option {key}: expected string, got {value!r}")
  return value


def get_opt_as_proto(raw, proto_type=ConfigProto):
  proto = proto_type()
  for key, value in Option(raw).items():
    setattr(proto, ALIASES.get(key, key), value)
  return proto


def proto_to_dict(proto):
  return {key: getattr(proto, key) for key in {**SCHEMA, **EXTENSIONS}}


def copy_proto(proto):
  new = type(proto)()
  for key, value in proto_to_dict(proto).items():
    setattr(new, key, value)
  return new


class Option(dict):
  """Options as a dict whose keys also read and write as attributes (``opt.max_m``); a missing key
  reads as None.  Positional arguments are dicts or names of JSON files (comments and trailing commas
  allowed); nested dicts become ``Option`` too.  Same behaviour as the reference's aux.Option."""

  def __init__(self, *sources, **fields):
    super().__init__()
    for src in sources:
      self.update(src if isinstance(src, dict) else load_json_file(src))
    self.update(fields)

  def update(self, other=(), **fields):  # route every entry through __setitem__
    for key, value in dict(other, **fields).items():
      self[key] = value

  def __setitem__(self, key, value):
    super().__setitem__(key, Option(value) if isinstance(value, dict) and not isinstance(value, Option) else value)

  def __getattr__(self, name):
    if name.startswith("__"):  # pickle and copy probe for dunder hooks
      raise AttributeError(name)
    return self.get(name)

  def __setattr__(self, name, value):
    self[name] = value

  def __delattr__(self, name):
    try:
      del self[name]
    except KeyError:
      raise AttributeError(name) from None
