"""The two-tile attention kernel (dh = 128, more than 128 query rows) against the CPU oracle and against the one-tile
kernel, through the C ABI.  Shapes chosen for its seams: a second tile that holds one row, sequence lengths that are not
multiples of 128 or 256, key ranges longer than the query range (the causal diagonal shifted by att - seq), grouped-query
heads, no mask, and q/o given token-major (strided heads) as the decoder layer holds them; few heads over long key ranges
(a tensor-parallel shard), where the key blocks of a tile pair are cut into runs that a second kernel merges.
Tolerance: max-abs 1e-2 on f16 outputs (convex combinations of N(0,1) values, |o| < ~4)."""
import numpy as np
import pytest
import torch

from helpers import assert_close
from test_gpu_mat_mul_attention import attention_case, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nh,nkvh,seq,att", [(4, 2, 129, 129), (4, 1, 256, 256), (8, 2, 1000, 1000), (4, 4, 513, 700), (2, 1, 384, 2000),
                                             (16, 4, 640, 640), (3, 3, 255, 255), (4, 1, 1536, 1536), (4, 2, 1100, 1300)])
def test_pair_kernel_shapes(pkg, orc, synth, dev, nh, nkvh, seq, att):
    attention_case(pkg, orc, synth, dev, nh, nkvh, seq, att, 128, True, seed=700, algos=("fused",))
    attention_case(pkg, orc, synth, dev, nh, nkvh, seq, att, 128, False, causal=False, seed=710, algos=("fused",))


def test_pair_kernel_agrees_with_one_tile_kernel(pkg, synth, dev):
    # same products, same exponentials, different schedule: the two fused kernels must agree to f16 rounding of the output
    nh, nkvh, seq, dh = 16, 4, 1536, 128
    q = to_dev(synth.normal(720, (nh, seq, dh), 1.0).astype(np.float16), dev)
    k = to_dev(synth.normal(721, (nkvh, seq, dh), 1.0).astype(np.float16), dev)
    v = to_dev(synth.normal(722, (nkvh, seq, dh), 1.0).astype(np.float16), dev)
    outs = []
    for algo in (pkg.ATTENTION_FUSED, pkg.ATTENTION_FUSED_ONE_TILE):
        op = pkg.Attention(0)
        op.set_algo(algo)
        o = torch.zeros_like(q)
        for rep in range(2):
            op.launch(pkg.AttentionArgs.of(q, k, v, o), torch.empty(16, dtype=torch.uint8, device=dev))
        torch.cuda.synchronize()
        assert op.status() == 0
        outs.append(o.cpu().numpy())
    assert_close(outs[0], outs[1], 4e-3, "two-tile vs one-tile kernel")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_key_block_runs_agree_with_whole_pairs(pkg, synth, dev, dtype):
    # 4 heads x 8 tile pairs = 32 CTAs: with a workspace the key blocks of every pair are cut into 4 runs (128 CTAs) whose
    # partial results a second kernel merges; without one each CTA finishes its rows itself.  Same products and the same
    # exponentials up to the reference point of each run: the outputs agree to the rounding of the 16-bit result.
    nh, nkvh, seq, att, dh = 4, 1, 2048, 2048 + 200, 128
    q = to_dev(synth.normal(730, (nh, seq, dh), 1.0).astype(np.float16), dev).to(dtype)
    k = to_dev(synth.normal(731, (nkvh, att, dh), 1.0).astype(np.float16), dev).to(dtype)
    v = to_dev(synth.normal(732, (nkvh, att, dh), 1.0).astype(np.float16), dev).to(dtype)
    outs = []
    for ws_bytes in (16, nh * seq * 4 * 528):
        op = pkg.Attention(0)
        o = torch.zeros_like(q)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        for rep in range(2):
            op.launch(pkg.AttentionArgs.of(q, k, v, o), ws)
        torch.cuda.synchronize()
        assert op.status() == 0
        outs.append(o.float().cpu().numpy())
    assert_close(outs[0], outs[1], 4e-3 if dtype == torch.float16 else 3e-2, "runs of key blocks vs whole pairs")
