from .numeric import calc_diff, count_bytes  # noqa: F401
from .bench import bench  # noqa: F401
