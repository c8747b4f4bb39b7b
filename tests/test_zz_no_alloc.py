"""The allocation-free random_sample entry point against the ordinary one, through the C ABI.

ops_random_sample_launch_noalloc exists for callers that cannot allocate device memory at the moment they
sample — a decode loop whose allocator is locked down, a plugin that receives a stream but no allocator, a
process with a fixed memory budget.  It takes no workspace: its scratch is a fixed array inside the library.
Because every call reuses that one array, the test calls it twice in a row (different rows, both modes) and
demands, bit for bit, what ops_random_sample_launch returns with a caller-provided workspace; a row longer
than the array is sized for must be refused with a clear error.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def kv_tuple(kv):
    return tuple(int(v) & 0xFFFFFFFF for v in kv.cpu().tolist())


def test_noalloc_matches_workspace_entry(pkg, synth, dev):
    op = pkg.RandomSample(0)
    rows = [synth.normal(0xB2000060 + i, (n,), 3.0).astype(dt) for i, (n, dt) in
            enumerate([(128256, np.float16), (32000, np.float32), (1, np.float16), (131072, np.float16)])]
    configs = [pkg.SampleArgs.arg_max(), pkg.SampleArgs(0.8, 0.9, 50), pkg.SampleArgs(2.5, 1.0, 2 ** 64 - 1)]
    for call in range(2):  # twice in a row: the second call starts from whatever the first left in the array
        for r, lg in enumerate(rows):
            x = torch.from_numpy(lg).to(dev)
            for c, cfg in enumerate(configs):
                seed = float(np.float32(0.137 + 0.29 * call + 0.11 * c))
                ws = torch.empty(16 * len(lg) + 256, dtype=torch.uint8, device=dev)
                want = torch.zeros(2, dtype=torch.int32, device=dev)
                op.launch(pkg.RandomSampleArgs.of(want, x, cfg, seed), ws)
                got = torch.full((2,), -1, dtype=torch.int32, device=dev)
                op.launch_noalloc(pkg.RandomSampleArgs.of(got, x, cfg, seed))
                torch.cuda.synchronize()
                assert kv_tuple(got) == kv_tuple(want), (call, r, c)  # bit-exact: index and value bits


def test_noalloc_refuses_rows_beyond_its_array(pkg, dev):
    op = pkg.RandomSample(0)
    limit = op.noalloc_max_logits()
    assert limit == 131072
    x = torch.zeros(limit + 8, dtype=torch.float16, device=dev)
    kv = torch.zeros(2, dtype=torch.int32, device=dev)
    with pytest.raises(pkg.LaunchError) as e:
        op.launch_noalloc(pkg.RandomSampleArgs.of(kv, x, pkg.SampleArgs(0.8, 0.9, 50), 0.5))
    assert e.value.kind == pkg.SHAPE_NOT_SUPPORT and str(limit) in e.value.info
    op.launch_noalloc(pkg.RandomSampleArgs.of(kv, x[:limit], pkg.SampleArgs(0.8, 0.9, 50), 0.5))  # exactly at the limit is fine
    torch.cuda.synchronize()
