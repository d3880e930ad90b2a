"""ctypes binding of the CPU oracle (oracle/libsfb_oracle.so) and of the reference's own
CPU operators (oracle/_ref/libsfb_ref.so).  Test infrastructure: only tests/, the smoke
check and the CPU-baseline leg of bench.py import this module."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

MASK_ALL, MASK_CAUSAL_DIAG, MASK_CAUSAL_ALL, MASK_LOCAL = 0, 1, 2, 3

_u8p = C.POINTER(C.c_uint8)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)


def build_oracle():
    """Compile the oracle (and the reference operators when the reference tree exists)."""
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)


def _ptr(a, t):
    return None if a is None else a.ctypes.data_as(t)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(ORACLE_DIR, "libsfb_oracle.so")
        if not os.path.exists(path):
            build_oracle()
        _lib = C.CDLL(path)
        _lib.orc_hash64.restype = C.c_uint64
        _lib.orc_hash64.argtypes = [C.c_uint64]
        _lib.orc_to_bhalf.restype = C.c_uint16
        _lib.orc_to_bhalf.argtypes = [C.c_float]
        _lib.orc_from_bhalf.restype = C.c_float
        _lib.orc_from_bhalf.argtypes = [C.c_uint16]
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def ref():
    """The reference's own CPU operators; None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        path = os.path.join(ORACLE_DIR, "_ref", "libsfb_ref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        _ref.ref_num_threads.restype = C.c_int
    return _ref


# ---------------------------------------------------------------- layouts
def layout(kind, heads, nb, **kw):
    out = np.zeros((heads, nb, nb), dtype=np.uint8)
    p = _ptr(out, _u8p)
    L = lib()
    if kind == "full":
        L.orc_layout_full(p, C.c_uint32(heads), C.c_uint32(nb), C.c_int(kw.get("causal", 0)))
    elif kind == "fixed":
        L.orc_layout_fixed(p, C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(kw.get("stride", 4)),
                           C.c_int(kw.get("causal", 0)))
    elif kind == "stride":
        L.orc_layout_stride(p, C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(kw.get("band", 4)),
                            C.c_uint32(kw.get("every", 8)), C.c_int(kw.get("causal", 0)))
    elif kind == "sawtooth":
        L.orc_layout_stride_sawtooth(p, C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(kw["chunks"]))
    elif kind == "local":
        L.orc_layout_local(p, C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(kw.get("left", 8)),
                           C.c_uint32(kw.get("right", 8)))
    elif kind == "bigbird":
        L.orc_layout_bigbird(p, C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(kw.get("window", 1)),
                             C.c_uint32(kw.get("g_first", 1)), C.c_uint32(kw.get("g_last", 1)),
                             C.c_uint32(kw.get("nrand", 3)), C.c_uint64(kw.get("seed", 1234)))
    else:
        raise ValueError(kind)
    return out


def lut_count(lay):
    heads, nb, _ = lay.shape
    blocks = C.c_uint32(0)
    rc = lib().orc_lut_count(_ptr(lay, _u8p), C.c_uint32(heads), C.c_uint32(nb), C.byref(blocks))
    if rc != 0:
        raise ValueError("heads have different block counts")
    return blocks.value


def lut_build(lay):
    """-> dict(nt, nn, rblk, nn_max, blocks) with uint32 arrays shaped [heads, n, 2]."""
    lay = np.ascontiguousarray(lay, dtype=np.uint8)
    heads, nb, _ = lay.shape
    blocks = lut_count(lay)
    nt = np.zeros((heads, blocks, 2), np.uint32)
    nn = np.zeros((heads, nb + blocks, 2), np.uint32)
    rb = np.zeros((heads, blocks, 2), np.uint32)
    mx = C.c_uint32(0)
    rc = lib().orc_lut_build(_ptr(lay, _u8p), C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(blocks),
                             _ptr(nt, _u32p), _ptr(nn, _u32p), _ptr(rb, _u32p), C.byref(mx))
    assert rc == 0
    return dict(nt=nt, nn=nn, rblk=rb, nn_max=mx.value, blocks=blocks)


def lut_build_tn(lay):
    """-> dict(tn [heads, nb+blocks, 2], tn_max, blocks): the LUT of the backward (TN) matmuls."""
    lay = np.ascontiguousarray(lay, dtype=np.uint8)
    heads, nb, _ = lay.shape
    blocks = lut_count(lay)
    tn = np.zeros((heads, nb + blocks, 2), np.uint32)
    mx = C.c_uint32(0)
    rc = lib().orc_lut_build_tn(_ptr(lay, _u8p), C.c_uint32(heads), C.c_uint32(nb), C.c_uint32(blocks),
                                _ptr(tn, _u32p), C.byref(mx))
    assert rc == 0
    return dict(tn=tn, tn_max=mx.value, blocks=blocks)


_WORD = {8: np.uint8, 16: np.uint16, 32: np.uint32, 64: np.uint64}


def mask_pack(nt, bs, pred, ctx=0):
    """-> (mask_np [heads, blocks, bs], mask_t [heads, bs, blocks]) of bs-bit words."""
    heads, blocks, _ = nt.shape
    wt = _WORD[bs]
    m_np = np.zeros((heads, blocks, bs), wt)
    m_t = np.zeros((heads, bs, blocks), wt)
    lib().orc_mask_pack(_ptr(nt, _u32p), C.c_uint32(heads), C.c_uint32(blocks), C.c_uint32(bs),
                        C.c_int(pred), C.c_uint32(ctx), m_np.ctypes.data_as(C.c_void_p),
                        m_t.ctypes.data_as(C.c_void_p))
    return m_np, m_t


# ---------------------------------------------------------------- arithmetic
def attention(q, k, v, luts, bs, scale, mask_np=None, eps=1e-6, round_s_bf16=False,
              want=("s", "p", "o")):
    """q,k,v float32 [B,L,H,d]; returns dict with the requested of s,p [B,H,blocks,bs,bs], o [B,L,H,d]."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    B, L, H, d = q.shape
    nb = L // bs
    nt, nn = luts["nt"], luts["nn"]
    blocks = luts["blocks"]
    lut_heads = nt.shape[0]
    mask_heads = 1 if mask_np is None else mask_np.shape[0]
    s = np.zeros((B, H, blocks, bs, bs), np.float32) if "s" in want else None
    p = np.zeros((B, H, blocks, bs, bs), np.float32) if "p" in want else None
    o = np.zeros((B, L, H, d), np.float32) if "o" in want else None
    lib().orc_attention(_ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(nt, _u32p), _ptr(nn, _u32p),
                        None if mask_np is None else mask_np.ctypes.data_as(C.c_void_p),
                        C.c_uint32(B), C.c_uint32(H), C.c_uint32(nb), C.c_uint32(bs), C.c_uint32(d),
                        C.c_uint32(blocks), C.c_uint32(lut_heads), C.c_uint32(mask_heads),
                        C.c_float(scale), C.c_float(eps), C.c_int(int(round_s_bf16)),
                        _ptr(s, _f32p), _ptr(p, _f32p), _ptr(o, _f32p))
    return dict(s=s, p=p, o=o)


def softmax_grad(dy, y, luts, bs, scale):
    """dy, y float32 [B,H,blocks,bs,bs] -> dx, same shape."""
    dy = np.ascontiguousarray(dy, np.float32)
    y = np.ascontiguousarray(y, np.float32)
    B, H, blocks, _, _ = dy.shape
    nn = luts["nn"]
    nb = nn.shape[1] - blocks
    dx = np.zeros_like(dy)
    lib().orc_softmax_grad(_ptr(dy, _f32p), _ptr(y, _f32p), _ptr(nn, _u32p), C.c_uint32(B), C.c_uint32(H),
                           C.c_uint32(nb), C.c_uint32(bs), C.c_uint32(blocks), C.c_uint32(nn.shape[0]),
                           C.c_float(scale), _ptr(dx, _f32p))
    return dx


def _spmm(fn, a, b, lut, bs):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    B, H, blocks, _, _ = a.shape
    _, L, _, d = b.shape
    c = np.zeros_like(b)
    fn(_ptr(a, _f32p), _ptr(b, _f32p), _ptr(lut, _u32p), C.c_uint32(B), C.c_uint32(H), C.c_uint32(L // bs),
       C.c_uint32(bs), C.c_uint32(d), C.c_uint32(blocks), C.c_uint32(lut.shape[0]), _ptr(c, _f32p))
    return c


def spmm_tn(a, b, tn, bs):
    """a [B,H,blocks,bs,bs], b [B,L,H,d] -> c [B,L,H,d] = A^T . B by block column."""
    return _spmm(lib().orc_spmm_tn, a, b, tn, bs)


def spmm_nn(a, b, nn, bs):
    """a [B,H,blocks,bs,bs], b [B,L,H,d] -> c [B,L,H,d] = A . B by block row."""
    return _spmm(lib().orc_spmm_nn, a, b, nn, bs)


def linear(x, w, bias=None, act=0):
    """out = act(x . w + bias), x [m,k], w [k,n]; act 1 = the reference's GELU."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    m, k = x.shape
    n = w.shape[1]
    out = np.zeros((m, n), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_linear(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(w, _f32p), None if b is None else _ptr(b, _f32p),
                     C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), C.c_int(act))
    return out


def linear_nt(x, wt, bias=None, act=0):
    """out = act(x . wt^T + bias), x [m,k], wt [n,k]."""
    x = np.ascontiguousarray(x, np.float32)
    wt = np.ascontiguousarray(wt, np.float32)
    m, k = x.shape
    n = wt.shape[0]
    out = np.zeros((m, n), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_linear_nt(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(wt, _f32p), None if b is None else _ptr(b, _f32p),
                        C.c_uint32(m), C.c_uint32(n), C.c_uint32(k), C.c_int(act))
    return out


def embedding(table, ids, pos=None):
    """table [vocab, hidden], ids int32 [B, L], pos [L, hidden] or None -> [B, L, hidden]."""
    table = np.ascontiguousarray(table, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    B, L = ids.shape
    vocab, hidden = table.shape
    out = np.zeros((B, L, hidden), np.float32)
    p = None if pos is None else np.ascontiguousarray(pos, np.float32)
    lib().orc_embedding(_ptr(out, _f32p), _ptr(table, _f32p), ids.ctypes.data_as(C.POINTER(C.c_int32)),
                        None if p is None else _ptr(p, _f32p), C.c_uint32(B), C.c_uint32(L), C.c_uint32(hidden), C.c_uint32(vocab))
    return out


def ref_embedding(table, ids, pos):
    """embedding_lookup + tensor_add_matrix of the reference (embedding.h:5-12, ewops.h:276-282)."""
    R = ref()
    assert R is not None
    table = np.ascontiguousarray(table, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    pos = np.ascontiguousarray(pos, np.float32)
    B, L = ids.shape
    hidden = table.shape[1]
    looked = np.zeros((B, L, hidden), np.float32)
    R.ref_embedding_lookup(_ptr(looked, _f32p), _ptr(table, _f32p), ids.ctypes.data_as(C.POINTER(C.c_int)), C.c_int(B), C.c_int(L),
                           C.c_int(1), C.c_int(hidden))
    out = np.zeros_like(looked)
    R.ref_tensor_add_matrix(_ptr(out, _f32p), _ptr(looked, _f32p), _ptr(pos, _f32p), C.c_int(B), C.c_int(L), C.c_int(hidden))
    return out


def ref_matmul_nt(a, b):
    """matrixMulNTCPU of the reference (matmul.h:121-132): a [m,k], b [n,k] -> a . b^T."""
    R = ref()
    assert R is not None
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    c = np.zeros((a.shape[0], b.shape[0]), np.float32)
    R.ref_matrixMulNTCPU(_ptr(c, _f32p), _ptr(a, _f32p), _ptr(b, _f32p), C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_int(b.shape[0]))
    return c


_i32p = C.POINTER(C.c_int32)


def csr_full_mask(L):
    rowptr = np.zeros(L + 1, np.int32)
    colidx = np.zeros(L * (L + 1) // 2, np.int32)
    lib().orc_csr_full_mask(rowptr.ctypes.data_as(_i32p), colidx.ctypes.data_as(_i32p), C.c_uint32(L))
    return rowptr, colidx


def csr_from_layout(lay2d, bs):
    lay2d = np.ascontiguousarray(lay2d, np.uint8)
    nb = lay2d.shape[0]
    rowptr = np.zeros(nb * bs + 1, np.int32)
    colidx = np.zeros(int(lay2d.sum()) * bs * bs, np.int32)
    fn = lib().orc_csr_from_layout
    fn.restype = C.c_uint32
    nnz = fn(_ptr(lay2d, _u8p), C.c_uint32(nb), C.c_uint32(bs), rowptr.ctypes.data_as(_i32p), colidx.ctypes.data_as(_i32p))
    assert nnz == colidx.size
    return rowptr, colidx


def csr_attention(q, k, v, rowptr, colidx, scale):
    q, k, v = (np.ascontiguousarray(t, np.float32) for t in (q, k, v))
    B, L, H, d = q.shape
    o = np.zeros_like(q)
    lib().orc_csr_attention(_ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), rowptr.ctypes.data_as(_i32p), colidx.ctypes.data_as(_i32p),
                            C.c_uint32(B), C.c_uint32(H), C.c_uint32(L), C.c_uint32(d), C.c_float(scale), _ptr(o, _f32p))
    return o


def ref_csr_full_mask(batch, heads, L):
    """generate_csr_full_mask of the reference (ewops.h:430-443) for batch*heads stacked patterns."""
    R = ref()
    assert R is not None
    rows = batch * heads * L
    rowptr = np.zeros(rows + 1, np.int32)
    colidx = np.zeros(batch * heads * L * (L + 1) // 2, np.int32)
    R.ref_generate_csr_full_mask(rowptr.ctypes.data_as(C.POINTER(C.c_int)), colidx.ctypes.data_as(C.POINTER(C.c_int)), C.c_int(batch),
                                 C.c_int(heads), C.c_int(L))
    return rowptr, colidx


def ref_matmul_nn(a, b):
    """matrixMulNNCPU of the reference (matmul.h:101-118)."""
    R = ref()
    assert R is not None
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    c = np.zeros((a.shape[0], b.shape[1]), np.float32)
    R.ref_matrixMulNNCPU(_ptr(c, _f32p), _ptr(a, _f32p), _ptr(b, _f32p), C.c_int(a.shape[0]), C.c_int(a.shape[1]), C.c_int(b.shape[1]))
    return c


def bias_residual_layernorm(x, bias, resid, gain, beta):
    x = np.ascontiguousarray(x, np.float32)
    m, hidden = x.shape
    out = np.zeros_like(x)
    summed = np.zeros_like(x)
    mean = np.zeros(m, np.float32)
    rstd = np.zeros(m, np.float32)
    f = lambda a: None if a is None else _ptr(np.ascontiguousarray(a, np.float32), _f32p)
    keep = [np.ascontiguousarray(a, np.float32) if a is not None else None for a in (bias, resid, gain, beta)]
    lib().orc_bias_residual_layernorm(_ptr(out, _f32p), _ptr(summed, _f32p), _ptr(mean, _f32p),
                                      _ptr(rstd, _f32p), _ptr(x, _f32p), _ptr(keep[0], _f32p),
                                      _ptr(keep[1], _f32p), _ptr(keep[2], _f32p), _ptr(keep[3], _f32p),
                                      C.c_uint32(m), C.c_uint32(hidden))
    return out, summed, mean, rstd


def bias_gelu(x, bias):
    x = np.ascontiguousarray(x, np.float32)
    m, n = x.shape
    out = np.zeros_like(x)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_bias_gelu(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(b, _f32p), C.c_uint32(m), C.c_uint32(n))
    return out


def ref_bias_gelu(x, bias):
    R = ref()
    assert R is not None
    x = np.ascontiguousarray(x, np.float32)
    m, n = x.shape
    t = np.zeros_like(x)
    R.ref_bias(_ptr(t, _f32p), _ptr(x, _f32p), _ptr(np.ascontiguousarray(bias, np.float32), _f32p), C.c_int(n), C.c_int(m))
    out = np.zeros_like(x)
    R.ref_gelu(_ptr(out, _f32p), _ptr(t, _f32p), C.c_int(1), C.c_int(m), C.c_int(n))
    return out


def magicu64(d):
    mg, sh = C.c_uint32(0), C.c_uint32(0)
    lib().orc_magicu64(C.c_uint32(d), C.byref(mg), C.byref(sh))
    return mg.value, sh.value


def fill_normal(shape, seed, stddev=1.0):
    out = np.empty(shape, np.float32)
    lib().orc_fill_normal(_ptr(out, _f32p), C.c_size_t(out.size), C.c_uint64(seed), C.c_float(stddev))
    return out


def to_bhalf(a):
    """fp32 array -> uint16 bf16 bits with the reference's rounding."""
    a = np.ascontiguousarray(a, np.float32)
    L = lib()
    return np.fromiter((L.orc_to_bhalf(C.c_float(float(x))) for x in a.ravel()), np.uint16, a.size).reshape(a.shape)


def from_bhalf(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------- reference CPU path
def ref_dense_causal_attention(q, k, v, scale):
    """The reference's own CPU attention (transformer_inference_part.cpp:219-224 order):
    transpose to [B,H,L,d], multiheadmatmulNT, softmax, multiheadmatmulNN, transpose back.
    Returns (scores [B,H,L,L], probs [B,H,L,L], o [B,L,H,d])."""
    R = ref()
    assert R is not None, "oracle/_ref/libsfb_ref.so not built"
    B, L, H, d = q.shape
    tq, tk, tv = (np.zeros((B, H, L, d), np.float32) for _ in range(3))
    for src, dst in ((q, tq), (k, tk), (v, tv)):
        src = np.ascontiguousarray(src, np.float32)
        R.ref_transpose_0123to0213(_ptr(src, _f32p), _ptr(dst, _f32p), C.c_int(B), C.c_int(L), C.c_int(H), C.c_int(d))
    s = np.zeros((B, H, L, L), np.float32)
    p = np.zeros((B, H, L, L), np.float32)
    R.ref_multiheadmatmulNT(_ptr(s, _f32p), _ptr(tq, _f32p), _ptr(tk, _f32p), C.c_int(B), C.c_int(H), C.c_int(L), C.c_int(d), C.c_int(L))
    R.ref_softmax(_ptr(p, _f32p), _ptr(s, _f32p), C.c_float(scale), C.c_int(L), C.c_int(B), C.c_int(H))
    to = np.zeros((B, H, L, d), np.float32)
    R.ref_multiheadmatmulNN(_ptr(to, _f32p), _ptr(p, _f32p), _ptr(tv, _f32p), C.c_int(B), C.c_int(H), C.c_int(L), C.c_int(L), C.c_int(d))
    o = np.zeros((B, L, H, d), np.float32)
    R.ref_transpose_0123to0213(_ptr(to, _f32p), _ptr(o, _f32p), C.c_int(B), C.c_int(H), C.c_int(L), C.c_int(d))
    return s, p, o


def ref_dense_backward(p, do, q, k, v, scale):
    """The reference's own CPU backward of attention (transformer.cpp:676-688 order) on dense [B,H,L,*]
    operands: dP = dO V^T, dV = P^T dO, dS = softmax_grad(dP, P), dQ = dS K, dK = dS^T Q.
    p [B,H,L,L]; do, q, k, v [B,H,L,d].  Returns (dp, ds, dq, dk, dv)."""
    R = ref()
    assert R is not None, "oracle/_ref/libsfb_ref.so not built"
    B, H, L, d = q.shape
    p, do, q, k, v = (np.ascontiguousarray(t, np.float32) for t in (p, do, q, k, v))
    i = C.c_int
    dp = np.zeros((B, H, L, L), np.float32)
    R.ref_multiheadmatmulNT(_ptr(dp, _f32p), _ptr(do, _f32p), _ptr(v, _f32p), i(B), i(H), i(L), i(d), i(L))
    dv = np.zeros((B, H, L, d), np.float32)
    R.ref_multiheadmatmulTN(_ptr(dv, _f32p), _ptr(p, _f32p), _ptr(do, _f32p), i(B), i(H), i(L), i(L), i(d))
    ds = np.zeros((B, H, L, L), np.float32)
    R.ref_softmax_grad(_ptr(ds, _f32p), _ptr(dp, _f32p), _ptr(p, _f32p), C.c_float(scale), i(B), i(H), i(L))
    dq = np.zeros((B, H, L, d), np.float32)
    R.ref_multiheadmatmulNN(_ptr(dq, _f32p), _ptr(ds, _f32p), _ptr(k, _f32p), i(B), i(H), i(L), i(L), i(d))
    dk = np.zeros((B, H, L, d), np.float32)
    R.ref_multiheadmatmulTN(_ptr(dk, _f32p), _ptr(ds, _f32p), _ptr(q, _f32p), i(B), i(H), i(L), i(L), i(d))
    return dp, ds, dq, dk, dv


def ref_bias_residual_layernorm(x, bias, resid, gain, beta):
    R = ref()
    assert R is not None
    x = np.ascontiguousarray(x, np.float32)
    m, hidden = x.shape
    t = np.zeros_like(x)
    R.ref_bias(_ptr(t, _f32p), _ptr(x, _f32p), _ptr(np.ascontiguousarray(bias, np.float32), _f32p), C.c_int(hidden), C.c_int(m))
    t2 = np.zeros_like(x)
    resid = np.ascontiguousarray(resid, np.float32)
    R.ref_tensor_add_tensor(_ptr(t2, _f32p), _ptr(resid, _f32p), _ptr(t, _f32p), C.c_int(1), C.c_int(m), C.c_int(hidden))
    out = np.zeros_like(x)
    mean = np.zeros(m, np.float32)
    rstd = np.zeros(m, np.float32)
    g = np.ascontiguousarray(gain, np.float32)
    b = np.ascontiguousarray(beta, np.float32)
    R.ref_layernorm(_ptr(out, _f32p), _ptr(mean, _f32p), _ptr(rstd, _f32p), _ptr(t2, _f32p), _ptr(g, _f32p), _ptr(b, _f32p), C.c_int(1), C.c_int(m), C.c_int(hidden))
    return out, t2, mean, rstd


def assert_close_16bit(got, ref, rel=2e-2, floor_of_rms=0.5):
    """Element-wise bar for results of 16-bit operands with fp32 accumulation: |got - ref| <= rel * |ref| + floor for every
    element, floor = rel * floor_of_rms * rms(ref).  The relative part is the stated 2e-2; the floor covers elements that are
    small only because their terms cancel (their error does not shrink with them: it is the rounding of the probabilities
    and of the exponentials' 16-bit arguments, about 1.5e-3 of rms(ref) per element, so the floor sits near six sigma)."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    floor = rel * floor_of_rms * float(np.sqrt(np.mean(ref * ref)))
    excess = np.abs(got - ref) - (rel * np.abs(ref) + floor)
    worst = float(excess.max())
    assert worst <= 0.0, "element-wise 16-bit bar exceeded by %g (floor %g)" % (worst, floor)


def blocks_to_dense(blk, nt, nb, bs):
    """[B,H,blocks,bs,bs] block tensor -> dense [B,H,L,L] (zeros elsewhere)."""
    B, H, blocks, _, _ = blk.shape
    out = np.zeros((B, H, nb * bs, nb * bs), blk.dtype)
    for h in range(H):
        lut = nt[h if nt.shape[0] > 1 else 0]
        for kk in range(blocks):
            i, j = int(lut[kk, 0]), int(lut[kk, 1])
            out[:, h, i * bs:(i + 1) * bs, j * bs:(j + 1) * bs] = blk[:, h, kk]
    return out


# ---------------------------------------------------------------- the reference's unfused GPU operators
_ref_gpu = None


def ref_gpu():
    """The reference's SDDMM / masked softmax / SpMM kernels compiled for this GPU
    (oracle/_ref/libsfb_ref_gpu.so); None when it was never built."""
    global _ref_gpu
    if _ref_gpu is None:
        path = os.path.join(ORACLE_DIR, "_ref", "libsfb_ref_gpu.so")
        if not os.path.exists(path):
            return None
        _ref_gpu = C.CDLL(path)
    return _ref_gpu


def split_layout(lay, factor=2):
    """The same element mask on blocks `factor` times smaller: every kept block becomes factor x factor kept blocks."""
    lay = np.ascontiguousarray(lay, dtype=np.uint8)
    return np.ascontiguousarray(lay.repeat(factor, axis=1).repeat(factor, axis=2))


class RefGpuAttention:
    """Device copies of the LUTs of one layout (built by the oracle, block size 32) and the three launches the
    reference's training driver makes per layer (transformer_attention_optimize.cu:728,738,748):
    bst_sgemm_nt -> BlocksparseMaskedSoftmax -> bst_sgemm_xn(NN_OP).  q, k, v: CUDA fp32 [B, L, H, d]."""

    def __init__(self, layout, device="cuda"):
        import torch
        self.torch = torch
        self.G = ref_gpu()
        assert self.G is not None
        luts = lut_build(layout)
        self.heads, self.nb = layout.shape[0], layout.shape[1]
        self.blocks, self.nn_max = luts["blocks"], luts["nn_max"]
        self.nt = torch.from_numpy(luts["nt"].view(np.int32)).to(device)
        self.nn = torch.from_numpy(luts["nn"].view(np.int32)).to(device)
        self.s = self.p = self.o = None

    def alloc(self, q, p_float=False):
        torch = self.torch
        B, L, H, d = q.shape
        assert L == self.nb * 32 and self.heads in (1, H) and q.dtype == torch.float32 and q.is_contiguous()
        self.s = torch.empty(B, H, self.blocks, 32, 32, dtype=torch.bfloat16, device=q.device)
        self.p = torch.empty(B, H, self.blocks, 32, 32, dtype=torch.float32 if p_float else torch.bfloat16, device=q.device)
        self.o = torch.empty_like(q)

    def launch(self, q, k, v, scale, marks=None):
        """The three launches on torch's current stream; returns nothing (results in self.s, self.p, self.o).
        marks: optional list of four CUDA events recorded before, between and after the launches."""
        torch = self.torch
        mark = (lambda i: marks[i].record()) if marks is not None else (lambda i: None)
        B, L, H, d = q.shape
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        vp = lambda t: C.c_void_p(t.data_ptr())
        u = C.c_uint32
        G = self.G
        mark(0)
        rc = G.ref_gpu_bst_sgemm_nt(st, vp(self.nt), vp(q), vp(k), vp(self.s), u(32), u(self.blocks), u(B), u(self.nb),
                                    u(self.nb), u(H), u(d), u(self.heads), u(self.blocks))
        assert rc == 0, rc
        mark(1)
        rc = G.ref_gpu_masked_softmax(st, vp(self.nn), None, vp(self.s), vp(self.p),
                                      C.c_int(1 if self.p.dtype == torch.float32 else 0), u(32), u(self.blocks), u(B),
                                      u(H), u(self.nb), u(self.heads), u(self.blocks + self.nb), u(self.nn_max),
                                      u(self.heads), C.c_float(scale))
        assert rc == 0, rc
        mark(2)
        if self.p.dtype == torch.bfloat16:
            rc = G.ref_gpu_bst_sgemm_nn(st, vp(self.nn), vp(self.p), vp(v), vp(self.o), u(32), u(self.blocks), u(B),
                                        u(self.nb), u(self.nb), u(H), u(d), u(self.heads), u(self.blocks + self.nb),
                                        u(self.nn_max))
            assert rc == 0, rc
        mark(3)
