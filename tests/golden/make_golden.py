"""Generate tests/golden/*.npz by running the UNMODIFIED reference on CPU.

The reference's Triton kernels run on the host under ``TRITON_INTERPRET=1``
(its own ops register for "cpu" in that mode, chill_attention/chill.py:60-62).
This script imports the reference from the directory given on the command line,
runs forward + backward on small seeded cases and stores inputs and outputs.
It is run once, where the reference checkout exists; the .npz files travel with
the repository, the reference does not.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

Cases (all fp32, inputs ~N(0,1) from torch.Generator().manual_seed(seed) drawn
in the order q, k, v, dO):
  c1_causal            CausalChillMask, (B,H,L,D) = (1,2,128,64)  - config 1 of the benchmark set
  full / sliding / chunkwise / prefixlm
                       the reference test-suite's mask parameters
                       (test/test_chill_attention.py:23-29) at (2,4,48,16) with
                       GQA (2 KV heads) and lens = [48, 21]
  sliding_rows         SlidingWindowChillMask(4,0), L=64, lens=[20,64]: the row
                       conventions (no visible key -> O=0, LSE=-inf; skipped
                       tile -> O=0, LSE=0)
  masks                make_mask(96) and both range tables for the five masks
"""
import os
import sys

assert os.environ.get("TRITON_INTERPRET") == "1", "run with TRITON_INTERPRET=1"
ref_dir = sys.argv[1]
sys.path.insert(0, ref_dir)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import chill_attention as ref  # noqa: E402

assert os.path.realpath(ref.__file__).startswith(os.path.realpath(ref_dir)), ref.__file__
out_dir = os.path.dirname(os.path.realpath(__file__))


def run_case(fname, mask, B, H, Hkv, L, D, seed, lens=None):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, L, D, generator=g)
    k = torch.randn(B, Hkv, L, D, generator=g)
    v = torch.randn(B, Hkv, L, D, generator=g)
    do = torch.randn(B, H, L, D, generator=g)
    lens_t = None if lens is None else torch.tensor(lens, dtype=torch.int32)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    o, lse = ref.chill_attention(qg, kg, vg, mask=mask, lens=lens_t, return_lse=True)
    o.backward(do)
    np.savez_compressed(
        os.path.join(out_dir, fname + ".npz"),
        mask_name=mask.name, mask_args=np.array(mask.constargs, dtype=np.int64),
        seed=seed, lens=np.array([] if lens is None else lens, dtype=np.int32),
        q=q.numpy(), k=k.numpy(), v=v.numpy(), do=do.numpy(),
        o=o.detach().numpy(), lse=lse.detach().numpy(),
        dq=qg.grad.numpy(), dk=kg.grad.numpy(), dv=vg.grad.numpy(),
    )
    print("wrote", fname, float(o.abs().max()))


run_case("c1_causal", ref.CausalChillMask(), 1, 2, 2, 128, 64, seed=21)
small = dict(B=2, H=4, Hkv=2, L=48, D=16, lens=[48, 21])
run_case("full", ref.FullChillMask(), seed=31, **small)
run_case("causal_small", ref.CausalChillMask(), seed=32, **small)
run_case("sliding", ref.SlidingWindowChillMask(10, 4), seed=33, **small)
run_case("chunkwise", ref.ChunkwiseChillMask(10, 4), seed=34, **small)
run_case("prefixlm", ref.PrefixLMChillMask(10), seed=35, **small)
run_case("sliding_rows", ref.SlidingWindowChillMask(4, 0), 2, 1, 1, 64, 16, seed=36, lens=[20, 64])

tables = {}
for m in (ref.FullChillMask(), ref.CausalChillMask(), ref.SlidingWindowChillMask(10, 4),
          ref.ChunkwiseChillMask(10, 4), ref.PrefixLMChillMask(10), ref.SlidingWindowChillMask(100, 0),
          ref.ChunkwiseChillMask(32, 2), ref.PrefixLMChillMask(40)):
    key = str(m).replace(" ", "")
    tables[key + "/mask"] = np.packbits(m.make_mask(96).cpu().numpy())
    tables[key + "/k_lims"] = m._calc_limits(96, m.k_range_for_q_jit).cpu().numpy()
    tables[key + "/q_lims"] = m._calc_limits(96, m.q_range_for_k_jit).cpu().numpy()
np.savez_compressed(os.path.join(out_dir, "masks.npz"), **tables)
print("wrote masks", sorted(tables))
