"""B200-native HNSW engine behind the Python API of cuhnsw (``from cuhnsw import CuHNSW``)."""
from cuhnsw_b200.pyhnsw import CuHNSW  # noqa: F401
