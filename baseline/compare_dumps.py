"""Element-wise comparison of the outputs the two builds of api_bench wrote (API_BENCH_DUMP=<prefix>):
python baseline/compare_dumps.py <prefix_a> <prefix_b>. Prints, per workload, whether the FP32 results are bitwise equal
and the largest difference relative to the largest magnitude."""
import glob
import os
import sys

import numpy as np

a, b = sys.argv[1], sys.argv[2]
for fa in sorted(glob.glob(a + "*.f32")):
    tag = fa[len(a):]
    fb = b + tag
    if not os.path.exists(fb):
        print(f"{tag}: missing in {b}")
        continue
    x, y = np.fromfile(fa, np.float32), np.fromfile(fb, np.float32)
    same = x.shape == y.shape and np.array_equal(x.view(np.uint32), y.view(np.uint32))
    diff = float(np.abs(x.astype(np.float64) - y).max() / max(np.abs(y).max(), 1e-30)) if x.shape == y.shape else float("nan")
    print(f"{tag[:-4]}: n={x.size} bitwise_equal={same} max_abs_diff_over_max={diff:.3e}")
