"""The floor under any kernel that hands a shared-memory stage from producer warps to an MMA
issuer once per item (tests/microbench/ring_handoff.cu): with nothing copied and nothing
multiplied the two-mbarrier hand-off alone costs a block about 300 clocks per item on B200,
whatever the ring depth, about 60 of them for releasing the stage with tcgen05.commit instead
of a plain arrive, and nothing for collecting one arrival per producer thread instead of one
per warp.  Four resident blocks overlap their hand-offs.  The test compiles the microbenchmark,
runs it (bounded waits, milliseconds of GPU time) and checks those orders of magnitude."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_handoff_cost_per_item(tmp_path):
    exe = str(tmp_path / "ring_handoff")
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-o", exe,
                           os.path.join(HERE, "microbench", "ring_handoff.cu")])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300).stdout
    rows = {}
    for line in out.splitlines():
        m = re.match(r"producer_warps=(\d+) stages=(\d+) ctas_per_sm=(\d+) full=(\w+) empty=(\w+) clk_per_item=([\d.]+) "
                     r"err=(\d)", line)
        assert m, line
        assert m.group(7) == "0", line
        rows[(int(m.group(1)), int(m.group(2)), int(m.group(3)), m.group(4), m.group(5))] = float(m.group(6))
    assert len(rows) == 10, out
    print(out)
    assert all(100 <= v <= 600 for v in rows.values()), rows
    # the ring depth does not change the cost: it is the issuer's own loop, not a round trip that stages could hide
    assert abs(rows[(8, 6, 1, "thread", "commit")] - rows[(8, 2, 1, "thread", "commit")]) <= 60, rows
    # an arrival per thread costs no more than an arrival per warp
    assert rows[(8, 6, 1, "thread", "commit")] <= rows[(8, 6, 1, "warp", "commit")] + 60, rows
