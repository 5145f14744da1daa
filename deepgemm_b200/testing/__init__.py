from .numeric import calc_diff, count_bytes, assert_bitwise_equal  # noqa: F401
from .bench import bench_events, get_arch_major  # noqa: F401
