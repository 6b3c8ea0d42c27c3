from . import bench, numeric, utils  # noqa: F401
from .numeric import calc_diff, count_bytes  # noqa: F401
from .bench import bench, bench_kineto  # noqa: F401
from .utils import assert_bitwise_equal, get_arch_major, ignore_env, test_filter  # noqa: F401
