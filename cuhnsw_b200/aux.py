"""Option handling and logging of the Python layer.

Mirrors cuhnsw/aux.py of the reference (get_logger :18-36, Option :79-119,
get_opt_as_proto :60-67, proto_to_dict :69-72).  The reference validates the
option dict by parsing it into a protobuf message generated from
cuhnsw/proto/config.proto; the generated module needs protoc, so the schema is
restated here as a typed table with the same field names, types and defaults,
and the same behaviour: unknown keys and wrongly typed values are rejected.
"""
import json
import logging
import re


def get_logger(name=__file__, level=2):
  if level == 1:
    level = logging.WARNING
  elif level == 2:
    level = logging.INFO
  elif level == 3:
    level = logging.DEBUG
  logger = logging.getLogger(name)
  if logger.handlers:
    return logger
  logger.setLevel(level)
  sh0 = logging.StreamHandler()
  sh0.setLevel(level)
  formatter = logging.Formatter("[%(levelname)-8s] %(asctime)s [%(filename)s] [%(funcName)s:%(lineno)d]"
                                "%(message)s", "%Y-%m-%d %H:%M:%S")
  sh0.setFormatter(formatter)
  logger.addHandler(sh0)
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
  "row_dtype": (str, "f32"),
}
ALIASES = {"heuristic_coff": "heuristic_coef"}


class ConfigProto:
  """Attribute bag with the fields of the reference's ConfigProto message."""

  def __init__(self):
    for key, (_, default) in {**SCHEMA, **EXTENSIONS}.items():
      object.__setattr__(self, key, default)

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
  """dict with attribute access; file names are loaded as JSON (aux.py:79-119)."""

  def __init__(self, *args, **kwargs):
    args = [arg if isinstance(arg, dict) else load_json_file(arg) for arg in args]
    super().__init__(*args, **kwargs)
    for arg in args:
      for k, val in arg.items():
        self[k] = Option(val) if isinstance(val, dict) else val
    for k, val in kwargs.items():
      self[k] = Option(val) if isinstance(val, dict) else val

  def __getattr__(self, attr):
    return self.get(attr)

  def __setattr__(self, key, value):
    self.__setitem__(key, value)

  def __setitem__(self, key, value):
    super().__setitem__(key, value)
    self.__dict__.update({key: value})

  def __delattr__(self, item):
    self.__delitem__(item)

  def __delitem__(self, key):
    super().__delitem__(key)
    del self.__dict__[key]

  def __getstate__(self):
    return vars(self)

  def __setstate__(self, state):
    vars(self).update(state)
