"""Generate tests/golden/decode_golden.npz from the REFERENCE's own CPU
implementation (oracle/_ref, built from the reference sources by
oracle/build_oracle.py). Inputs are regenerated from seeds by tests/cases.py,
so the fixture stores outputs only plus a checksum of each input set.

    python tests/golden/make_golden.py

Needs the reference checkout (to build oracle/_ref); the parity tests then
run anywhere from the committed fixture.
"""

import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
import oracle  # noqa: E402
from oracle import build_oracle  # noqa: E402


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64)[0]


def main():
    build_oracle.build_oracle()
    if build_oracle.build_ref() is None:
        raise SystemExit("no reference checkout: cannot generate golden vectors")
    out = {}
    for (b, hq, hkv, t, d, wl) in cases.SHAPES:
        rng = np.random.default_rng(cases.shape_seed(b, hq, hkv, t, d))
        q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, wl)
        name = "shape_%d_%d_%d_%d_%d" % (b, hq, hkv, t, d)
        out[name] = oracle.ref_decode(q, k, v, lens)
        out[name + "_sum"] = digest(q, k, v, lens)
    for name, (seed, b, hq, hkv, d, nb, lens) in cases.PAGED_CASES.items():
        rng = np.random.default_rng(seed)
        q, kp, vp, tbl, kc, vc, la = cases.make_paged_case(rng, b, hq, hkv, d, nb, lens)
        out[name] = oracle.ref_decode_paged(q, kp, vp, tbl, la)
        out[name + "_sum"] = digest(q, kp, vp, tbl, la)
    # benchmark configuration 1 in full, configuration 2 reduced (fp32 values
    # and the bf16-rounded values the half-precision kernels actually see)
    q, k, v = cases.config1()
    out["config1"] = oracle.ref_decode(q, k, v)
    out["config1_sum"] = digest(q, k, v)
    import torch
    q, k, v = cases.config2(batch=1, t=1024)
    qr, kr, vr = (cases.round_to(x, torch.bfloat16) for x in (q, k, v))
    out["config2_b1_t1024_bf16"] = oracle.ref_decode(qr, kr, vr)
    out["config2_b1_t1024_bf16_sum"] = digest(qr, kr, vr)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "decode_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "entries")

    # prefill: full outputs for the small shapes, a digest of the output bytes for the large ones
    # (parity of the restatement is bit-exact, so a digest pins it just as well)
    pre = {}
    for (b, hq, hkv, s, d) in cases.PREFILL_SHAPES:
        for causal in (True, False):
            q, k, v = cases.make_prefill_case(b, hq, hkv, s, d, causal)
            y = oracle.ref_prefill(q, k, v, causal)
            name = "prefill_%d_%d_%d_%d_%d_%d" % (b, hq, hkv, s, d, int(causal))
            if y.size <= 20000:
                pre[name] = y
            pre[name + "_out_sum"] = digest(y)
            pre[name + "_sum"] = digest(q, k, v)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "prefill_golden.npz")
    np.savez_compressed(path, **pre)
    print("wrote", path, os.path.getsize(path), "bytes,", len(pre), "entries")


if __name__ == "__main__":
    main()
