"""Regenerates tests/golden/ref_uploads.npz, tests/golden/ref_cpu_attention.npz and tests/golden/ref_cpu_backward.npz.

Needs the reference tree (read-only) and a C/CUDA toolchain, but no GPU:

  python tests/golden/make_golden.py [/path/to/reference]

1. ref_uploads.npz -- the reference's own test programs (stride / local / big_bird /
   no_fusion *_test.cu) are compiled unmodified and linked against oracle/fake_cudart.c,
   a stand-in runtime that launches nothing and records every host->device upload.  The
   uploads are the nt_lut / nn_lut / mask / rblk_lut arrays those programs build, plus the
   launch geometry of each kernel.  fixed_fusion_test.cu is left out: it sizes its arrays
   from a variable it never initialises (fixed_fusion_test.cu:46,109-115) and crashes.
2. ref_cpu_attention.npz -- outputs of the reference's own CPU operators (matmul.h,
   ewops.h, layernorm.h through oracle/_ref/libsfb_ref.so) on small seeded inputs.
3. ref_cpu_backward.npz -- the same operators run in the backward order of transformer.cpp:676-688
   (multiheadmatmulNT, multiheadmatmulTN, softmax_grad, multiheadmatmulNN, multiheadmatmulTN).
"""
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))

# order of the uploads inside each program (names are ours)
UPLOADS = {
    "stride_fusion_test": ["nt_lut", "nn_lut", "mask_np", "mask_t", None, None, "rblk_lut"],
    "local_fusion_test": ["nt_lut", "nn_lut", "mask_np", "mask_t", None, None, "rblk_lut"],
    "no_fusion_test": ["nt_lut", "nn_lut", "mask_np", "mask_t", None, None],
    "big_bird_fusion_test": ["nt_lut", "nn_lut", None, None, "rblk_lut"],
}


def capture(ref):
    subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "REF=" + ref, "all", "capture"], check=True)
    out = {}
    for test, names in UPLOADS.items():
        with tempfile.TemporaryDirectory() as tmp:
            env = dict(os.environ, SFB_CAPTURE_DIR=tmp)
            subprocess.run([os.path.join(ROOT, "oracle", "_ref", "capture_" + test)], cwd=tmp, env=env,
                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, check=True, timeout=600)
            log = open(os.path.join(tmp, "capture.log")).read().splitlines()
            sizes = [int(l.split()[3]) for l in log if l.startswith("h2d")]
            assert len(sizes) == len(names), (test, sizes)
            for i, name in enumerate(names):
                if name is None:
                    continue
                raw = np.fromfile(os.path.join(tmp, "h2d_%02d.bin" % i), dtype=np.uint32)
                assert raw.nbytes == sizes[i]
                out[test + "/" + name] = raw
            launches = [l for l in log if l.startswith("launch")]
            geo = []
            for l in launches:
                m = re.match(r"launch (\S+) grid (\d+) (\d+) (\d+) block (\d+) (\d+) (\d+) smem (\d+)", l)
                geo.append(m.group(1) + " " + " ".join(m.group(i) for i in range(2, 9)))
            out[test + "/launches"] = np.array(geo)
    return out


def cpu_reference():
    import oracle_lib as O
    out = {}
    B, L, H, d = 2, 96, 3, 64
    q = O.fill_normal((B, L, H, d), 11)
    k = O.fill_normal((B, L, H, d), 12)
    v = O.fill_normal((B, L, H, d), 13)
    scale = np.float32(1.0 / np.sqrt(d))
    s, p, o = O.ref_dense_causal_attention(q, k, v, scale)
    out["attn/shape"] = np.array([B, L, H, d])
    out["attn/seeds"] = np.array([11, 12, 13])
    out["attn/s"] = s
    out["attn/p"] = p
    out["attn/o"] = o
    m, hidden = 48, 768
    x = O.fill_normal((m, hidden), 21)
    r = O.fill_normal((m, hidden), 22)
    b = O.fill_normal((hidden,), 23, 0.02)
    g = 1.0 + O.fill_normal((hidden,), 24, 0.1)
    be = O.fill_normal((hidden,), 25, 0.1)
    y, summed, mean, rstd = O.ref_bias_residual_layernorm(x, b, r, g, be)
    out["ln/shape"] = np.array([m, hidden])
    out["ln/seeds"] = np.array([21, 22, 23, 24, 25])
    out["ln/y"] = y
    out["ln/sum"] = summed
    out["ln/mean"] = mean
    out["ln/rstd"] = rstd
    return out


def cpu_reference_backward():
    """Backward of attention by the reference's own CPU operators (transformer.cpp:676-688): the forward
    probabilities come from the same operators, dO from the seeded generator."""
    import oracle_lib as O
    B, L, H, d = 1, 96, 2, 32
    q, k, v, do = (O.fill_normal((B, L, H, d), s) for s in (41, 42, 43, 44))
    scale = np.float32(1.0 / np.sqrt(d))
    _, p, _ = O.ref_dense_causal_attention(q, k, v, scale)
    t = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3))     # [B,L,H,d] -> [B,H,L,d]
    dp, ds, dq, dk, dv = O.ref_dense_backward(p, t(do), t(q), t(k), t(v), scale)
    return {"bwd/shape": np.array([B, L, H, d]), "bwd/seeds": np.array([41, 42, 43, 44]), "bwd/p": p, "bwd/dp": dp,
            "bwd/ds": ds, "bwd/dq": dq, "bwd/dk": dk, "bwd/dv": dv}


if __name__ == "__main__":
    # the reference tree: first argument, else SFB_REFERENCE_DIR, else a directory `reference` beside this repository
    ref = (sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SFB_REFERENCE_DIR")
           or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
    np.savez_compressed(os.path.join(HERE, "ref_uploads.npz"), **capture(ref))
    np.savez_compressed(os.path.join(HERE, "ref_cpu_attention.npz"), **cpu_reference())
    np.savez_compressed(os.path.join(HERE, "ref_cpu_backward.npz"), **cpu_reference_backward())
    print("wrote", os.listdir(HERE))
