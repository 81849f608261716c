"""Regenerate the golden vectors in this folder from the reference's own Python package.

Run in a checkout where the reference tree is mounted:

    python tests/golden/make_golden.py [/path/to/reference]

Writes compressed ``.npz`` files beside this script:

* ``ref_<name>.npz``      the four fixtures the reference commits under
                          ``reference/tests/fixtures/*.pt`` (config, q, k, v, out),
                          converted without change (``reference/tests/test_golden.py:40-91``);
* ``gen_prefill_*.npz``   fresh outputs of ``ring_attention_ref.ring_attention``
                          (``reference/ring_attention_ref/ring.py:18-70``) for the layouts the
                          committed fixtures do not cover: striped, zig-zag with n_splits=4,
                          head_dim 64/128, plus the per-rank index maps;
* ``gen_decode_*.npz``    a prefill + decode trajectory from
                          ``ring_attention_ref.inference`` (``inference.py:74-216``);
* ``index_maps.npz``      ``zigzag_indices`` / ``striped_indices`` tables
                          (``zigzag.py:12-92``).

The test-suite only reads the ``.npz`` files; it never imports the reference.
"""
import os
import sys

import numpy as np
import torch

_BESIDE_REPO = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))
REF = sys.argv[1] if len(sys.argv) > 1 else _BESIDE_REPO
sys.path.insert(0, os.path.join(REF, "reference"))
HERE = os.path.dirname(os.path.abspath(__file__))

from ring_attention_ref import ring_attention  # noqa: E402
from ring_attention_ref.inference import decode_step, prefill  # noqa: E402
from ring_attention_ref.zigzag import striped_indices, zigzag_indices  # noqa: E402


def save(name, **arrs):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: (v.numpy() if torch.is_tensor(v) else np.asarray(v))
                                 for k, v in arrs.items()})
    print("wrote", path, os.path.getsize(path))


def main():
    fx = os.path.join(REF, "reference", "tests", "fixtures")
    for f in sorted(os.listdir(fx)):
        if not f.endswith(".pt"):
            continue
        d = torch.load(os.path.join(fx, f), weights_only=False)
        c = d["config"]
        save("ref_" + f[:-3], q=d["q"], k=d["k"], v=d["v"], out=d["out"],
             cp_size=c["cp_size"], causal=int(c["causal"]), zig_zag=int(c["zig_zag"]),
             seed=c["seed"])

    cases = [
        # name, B, H, S, D, cp, causal, zigzag, n_splits, striped, seed
        ("striped_cp4_d64", 1, 2, 128, 64, 4, True, False, 2, True, 11),
        ("zigzag4_cp2_d64", 1, 2, 128, 64, 2, True, True, 4, False, 12),
        ("zigzag_cp4_d128", 1, 1, 256, 128, 4, True, True, 2, False, 13),
        ("contig_cp2_d128", 2, 1, 128, 128, 2, True, False, 2, False, 14),
    ]
    for name, B, H, S, D, cp, causal, zz, ns, st, seed in cases:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn((B, H, S, D), generator=g)
        k = torch.randn((B, H, S, D), generator=g)
        v = torch.randn((B, H, S, D), generator=g)
        out = ring_attention(q, k, v, cp_size=cp, causal=causal, zig_zag=zz, n_splits=ns, striped=st)
        if zz:
            idx = zigzag_indices(S, cp_size=cp, n_splits=ns)
        elif st:
            idx = striped_indices(S, cp_size=cp)
        else:
            idx = torch.arange(S).reshape(cp, S // cp)
        save("gen_prefill_" + name, q=q, k=k, v=v, out=out, idx=idx, cp_size=cp, causal=int(causal))

    # prefill + 6 decode steps, round-robin owner, cp=2, MHA (the reference is MHA-only here)
    B, H, S, D, cp, steps = 2, 4, 64, 64, 2, 6
    g = torch.Generator().manual_seed(21)
    q = torch.randn((B, H, S, D), generator=g)
    k = torch.randn((B, H, S, D), generator=g)
    v = torch.randn((B, H, S, D), generator=g)
    out_shards, cache = prefill(q, k, v, cp_size=cp, causal=True, zig_zag=False,
                                s_max=S // cp + steps)
    qs, ks, vs, outs = [], [], [], []
    for t in range(steps):
        qn = torch.randn((B, H, 1, D), generator=g)
        kn = torch.randn((B, H, 1, D), generator=g)
        vn = torch.randn((B, H, 1, D), generator=g)
        o, cache = decode_step(qn, kn, vn, cache, owner_rank=t % cp)
        qs.append(qn); ks.append(kn); vs.append(vn); outs.append(o)
    save("gen_decode_cp2", q=q, k=k, v=v, prefill_out=out_shards, dq=torch.stack(qs),
         dk=torch.stack(ks), dv=torch.stack(vs), dout=torch.stack(outs), cp_size=cp)

    save("index_maps",
         zz_16_2=zigzag_indices(16, 2), zz_32_4=zigzag_indices(32, 4),
         zz_32_2_n4=zigzag_indices(32, 2, n_splits=4), zz_48_3=zigzag_indices(48, 3),
         st_16_4=striped_indices(16, 4), st_12_3=striped_indices(12, 3))


if __name__ == "__main__":
    main()
