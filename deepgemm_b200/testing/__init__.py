from .numeric import calc_diff, count_bytes, assert_bitwise_equal  # noqa: F401
from .bench import bench, bench_events, bench_kineto, get_arch_major, test_filter  # noqa: F401
