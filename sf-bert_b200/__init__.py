"""Python host side of libsfbert_b200.so: a ctypes binding of the C ABI (include/sfbert_b200.h)
plus thin helpers that mirror the reference's operator surface (blocksparse.h,
fusion_blocksparse.h) on torch tensors.  torch is used for device memory and streams only;
every operator below runs a hand-written sm_100a kernel from the shared library, and the import
fails loudly when the library is missing -- there is no fallback."""
import ctypes as C
import math
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SFBERT_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("SFBERT_B200_LIB") or os.path.join(_HERE, "libsfbert_b200.so")

F32, BF16, F16 = 0, 1, 2
LAYOUT_FULL, LAYOUT_FIXED, LAYOUT_STRIDE, LAYOUT_SAWTOOTH, LAYOUT_LOCAL, LAYOUT_BIGBIRD = range(6)
MASK_ALL, MASK_CAUSAL_DIAG, MASK_CAUSAL_ALL, MASK_LOCAL = range(4)
NT_OP, NN_OP, TN_OP = 0, 1, 2
ACT_NONE, ACT_GELU = 0, 1

# every symbol include/sfbert_b200.h declares
SYMBOLS = [
    "sfb_last_error", "sfb_version", "sfb_layout_generate", "sfb_lut_count", "sfb_lut_build", "sfb_mask_pack",
    "sfb_magicu64", "sfb_bst_sgemm_nt", "sfb_masked_softmax", "sfb_bst_sgemm_xn", "sfb_fused_sddmm_softmax",
    "sfb_fused_attention", "sfb_bias_residual_layernorm", "sfb_device_status", "sfb_bias_gelu", "sfb_lut_build_tn",
    "sfb_masked_softmax_grad", "sfb_linear", "sfb_linear_nt", "sfb_embedding", "sfb_csr_from_layout",
    "sfb_csr_attention", "sfb_rowdot", "sfb_fused_sddmm_softmax_grad", "sfb_fused_attention_slice", "sfb_device_status_clear",
]

if not os.path.exists(LIB_PATH):
    raise ImportError("%s is missing: build it with `make -C %s/csrc` (needs nvcc, sm_100a)" % (LIB_PATH, _HERE))
lib = C.CDLL(LIB_PATH)
lib.sfb_last_error.restype = C.c_char_p
for _name in SYMBOLS:
    getattr(lib, _name)

_u32, _i32, _u64, _f32, _vp = C.c_uint32, C.c_int, C.c_uint64, C.c_float, C.c_void_p
lib.sfb_layout_generate.argtypes = [_vp, _vp, _u32, _u32, _i32, _u32, _u32, _u32, _u32, _i32, _u64]
lib.sfb_lut_count.argtypes = [_vp, _vp, _u32, _u32, _vp]
lib.sfb_lut_build.argtypes = [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp]
lib.sfb_mask_pack.argtypes = [_vp, _vp, _u32, _u32, _u32, _i32, _u32, _vp, _vp]
lib.sfb_magicu64.argtypes = [_u32, C.POINTER(_u32), C.POINTER(_u32)]
lib.sfb_magicu64.restype = None
lib.sfb_bst_sgemm_nt.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32, _i32] + [_u32] * 9
lib.sfb_masked_softmax.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32, _i32] + [_u32] * 9 + [_f32]
lib.sfb_bst_sgemm_xn.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32, _i32] + [_u32] * 13
lib.sfb_lut_build_tn.argtypes = [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp]
lib.sfb_masked_softmax_grad.argtypes = [_vp, _vp, _vp, _vp, _vp, _i32] + [_u32] * 8 + [_f32]
lib.sfb_linear.argtypes = [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _i32, _i32]
lib.sfb_linear_nt.argtypes = [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _i32, _i32]
lib.sfb_embedding.argtypes = [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _i32, _vp]
lib.sfb_csr_from_layout.argtypes = [_vp, _vp, _u32, _u32, _vp, _vp]
lib.sfb_rowdot.argtypes = [_vp, _vp, _vp, _vp, _u64, _u32, _i32]
lib.sfb_fused_sddmm_softmax_grad.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32] + [_u32] * 8 + [_f32]
lib.sfb_csr_attention.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _u32, _u32, _u32, _u32, _f32, _vp]
lib.sfb_fused_sddmm_softmax.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32] + [_u32] * 10 + [_f32]
lib.sfb_fused_attention.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32] + [_u32] * 9 + [_f32, _u32]
lib.sfb_fused_attention_slice.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32] + [_u32] * 9 + [_f32, _u32, _u64, _u64]
lib.sfb_bias_residual_layernorm.argtypes = [_vp] * 10 + [_u32, _u32, _i32]


lib.sfb_device_status.argtypes = [C.POINTER(_u32)]
lib.sfb_bias_gelu.argtypes = [_vp, _vp, _vp, _vp, _u32, _u32, _i32]


def device_status():
    """0 unless a kernel gave up on one of its bounded waits (synchronises with the device)."""
    v = _u32(0)
    _check(lib.sfb_device_status(C.byref(v)))
    return v.value


def device_status_clear():
    """Sets the status word back to 0 (synchronises with the device)."""
    _check(lib.sfb_device_status_clear())


class SfbError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise SfbError(lib.sfb_last_error().decode())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def dtype_tag(t):
    return _DT[t.dtype]


def magicu64(d):
    """magicu64 of blocksparse.h:1016-1043."""
    m, s = _u32(0), _u32(0)
    lib.sfb_magicu64(d, C.byref(m), C.byref(s))
    return m.value, s.value


class BlockLayout:
    """A block layout and its look-up tables in device memory (what the reference's test programs
    build on the host and upload, stride_fusion_test.cu:48-227)."""

    def __init__(self, layout, block_size):
        assert layout.dtype == torch.uint8 and layout.dim() == 3 and layout.is_cuda
        self.layout = layout.contiguous()
        self.heads, self.nb, _ = layout.shape
        self.block_size = block_size
        dev = layout.device
        counts = torch.zeros(self.heads, dtype=torch.int32, device=dev)
        _check(lib.sfb_lut_count(_stream(), _p(self.layout), self.heads, self.nb, _p(counts)))
        counts = counts.cpu()  # the one host read: sizes the tables
        if int(counts.min()) != int(counts.max()):
            raise SfbError("heads have different block counts: %s" % counts.tolist())
        self.blocks = int(counts[0])
        self.nt_lut = torch.zeros(self.heads, self.blocks, 2, dtype=torch.int32, device=dev)
        self.nn_lut = torch.zeros(self.heads, self.nb + self.blocks, 2, dtype=torch.int32, device=dev)
        self.rblk_lut = torch.zeros(self.heads, self.blocks, 2, dtype=torch.int32, device=dev)
        nn_max = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        _check(lib.sfb_lut_build(_stream(), _p(self.layout), self.heads, self.nb, self.blocks, _p(self.nt_lut),
                                 _p(self.nn_lut), _p(self.rblk_lut), _p(nn_max), _p(status)))
        if int(status.item()) != 0:
            raise SfbError("sfb_lut_build: block count mismatch")
        self.nn_max = int(nn_max.item())
        self.mask_np = None
        self.mask_t = None
        self._tn = None

    def _build_tn(self):
        """The column-major LUT of the backward matmuls, built on first use."""
        if self._tn is None:
            dev = self.layout.device
            tn = torch.zeros(self.heads, self.nb + self.blocks, 2, dtype=torch.int32, device=dev)
            tn_max = torch.zeros(1, dtype=torch.int32, device=dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            _check(lib.sfb_lut_build_tn(_stream(), _p(self.layout), self.heads, self.nb, self.blocks, _p(tn), _p(tn_max),
                                        _p(status)))
            if int(status.item()) != 0:
                raise SfbError("sfb_lut_build_tn: block count mismatch")
            self._tn = (tn, int(tn_max.item()))
        return self._tn

    @property
    def tn_lut(self):
        return self._build_tn()[0]

    @property
    def tn_max(self):
        return self._build_tn()[1]

    @classmethod
    def generate(cls, kind, heads, nb, block_size, p0=0, p1=0, p2=0, p3=0, causal=0, seed=0, device="cuda"):
        lay = torch.empty(heads, nb, nb, dtype=torch.uint8, device=device)
        _check(lib.sfb_layout_generate(_stream(), _p(lay), heads, nb, kind, p0, p1, p2, p3, causal, seed))
        return cls(lay, block_size)

    def pack_mask(self, pred, ctx=0):
        wt = torch.int32 if self.block_size == 32 else torch.int64
        dev = self.layout.device
        self.mask_np = torch.zeros(self.heads, self.blocks, self.block_size, dtype=wt, device=dev)
        self.mask_t = torch.zeros(self.heads, self.block_size, self.blocks, dtype=wt, device=dev)
        _check(lib.sfb_mask_pack(_stream(), _p(self.nt_lut), self.heads, self.blocks, self.block_size, pred, ctx,
                                 _p(self.mask_np), _p(self.mask_t)))
        return self

    @property
    def nt_lut_dim(self):
        return self.blocks

    @property
    def nn_lut_dim(self):
        return self.blocks + self.nb


def _dims(q, lay):
    B, L, H, d = q.shape
    assert L == lay.nb * lay.block_size, "sequence length does not match the layout"
    assert lay.heads in (1, H)
    return B, L, H, d


def bst_sgemm_nt(q, k, lay, out_dtype=torch.bfloat16):
    """S = Q.K^T on the kept blocks, unscaled (bst_sgemm_nt / bst_sgemm_nt_float, blocksparse.h:425,202)."""
    B, L, H, d = _dims(q, lay)
    s = torch.empty(B, H, lay.blocks, lay.block_size, lay.block_size, dtype=out_dtype, device=q.device)
    _check(lib.sfb_bst_sgemm_nt(_stream(), _p(lay.nt_lut), _p(q), _p(k), _p(s), dtype_tag(q), _DT[out_dtype],
                                lay.block_size, lay.blocks, B, lay.nb, lay.nb, H, d, lay.heads, lay.nt_lut_dim))
    return s


def masked_softmax(s, lay, scale, out_dtype=torch.bfloat16, use_mask=False):
    """BlocksparseMaskedSoftmax<T,V> (blocksparse.h:649-722)."""
    B, H = s.shape[:2]
    y = torch.empty(s.shape, dtype=out_dtype, device=s.device)
    mask = lay.mask_t if use_mask else None
    _check(lib.sfb_masked_softmax(_stream(), _p(lay.nn_lut), _p(mask), _p(s), _p(y), dtype_tag(s), _DT[out_dtype],
                                  lay.block_size, lay.blocks, B, H, lay.nb, lay.heads, lay.nn_lut_dim, lay.nn_max,
                                  lay.heads, scale))
    return y


def bst_sgemm_xn(p, v, lay):
    """O = P.V over each block-row (bst_sgemm_xn with NN_OP, blocksparse.h:965-1014)."""
    B, L, H, d = _dims(v, lay)
    o = torch.empty_like(v)
    magic, shift = magicu64((d + 63) // 64)
    _check(lib.sfb_bst_sgemm_xn(_stream(), _p(lay.nn_lut), _p(p), _p(v), _p(o), dtype_tag(p), dtype_tag(v), lay.block_size,
                                lay.blocks, B, lay.nb, lay.nb, H, d, lay.heads, lay.nn_lut_dim, NN_OP, magic, shift,
                                lay.nn_max))
    return o


def linear(x, w, bias=None, act=ACT_NONE, out=None):
    """out = act(x . w + bias) on the tensor cores: x [..., k], w [k, n] row-major, 16-bit; bias fp32 [n].
    The projections of the encoder layer with their bias add / GELU folded in
    (transformer_attention_optimize.cu:693-716, 755-763, 773-793)."""
    k, n = w.shape
    assert x.shape[-1] == k and x.dtype == w.dtype and x.is_contiguous() and w.is_contiguous()
    m = x.numel() // k
    o = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device) if out is None else out
    _check(lib.sfb_linear(_stream(), _p(o), _p(x), _p(w), _p(bias), m, n, k, dtype_tag(x), act))
    return o


def linear_nt(x, wt, bias=None, act=ACT_NONE, out=None):
    """out = act(x . wt^T + bias) with wt [n, k] row-major: the logits over the tied embedding table
    (transformer_inference_part.cpp:241)."""
    n, k = wt.shape
    assert x.shape[-1] == k and x.dtype == wt.dtype and x.is_contiguous() and wt.is_contiguous()
    m = x.numel() // k
    o = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device) if out is None else out
    _check(lib.sfb_linear_nt(_stream(), _p(o), _p(x), _p(wt), _p(bias), m, n, k, dtype_tag(x), act))
    return o


def embedding(table, ids, pos=None):
    """out[b, l, :] = table[ids[b, l], :] + pos[l, :] (embedding_lookup + tensor_add_matrix, embedding.h:5-12,
    ewops.h:276-282).  Returns (out, number of ids that were outside the table)."""
    B, L = ids.shape
    vocab, hidden = table.shape
    assert ids.dtype == torch.int32 and ids.is_contiguous() and table.is_contiguous()
    out = torch.empty(B, L, hidden, dtype=table.dtype, device=table.device)
    bad = torch.empty(1, dtype=torch.int32, device=table.device)      # the call zeroes it on the stream
    _check(lib.sfb_embedding(_stream(), _p(out), _p(table), _p(ids), _p(pos), B, L, hidden, vocab, dtype_tag(table), _p(bad)))
    return out, bad


def csr_from_layout(lay, head=0):
    """(rowptr, colidx): the element pattern of one head of a BlockLayout as CSR (every element of every kept block)."""
    bs, nb = lay.block_size, lay.nb
    dev = lay.layout.device
    rowptr = torch.empty(nb * bs + 1, dtype=torch.int32, device=dev)
    colidx = torch.empty(lay.blocks * bs * bs, dtype=torch.int32, device=dev)
    _check(lib.sfb_csr_from_layout(_stream(), _p(lay.layout[head]), nb, bs, _p(rowptr), _p(colidx)))
    return rowptr, colidx


def csr_attention(q, k, v, rowptr, colidx, scale):
    """Element-sparse attention over one CSR pattern shared by every (batch, head) (the reference's csr_* prototype,
    cuda_kernels.h:976-1075).  Returns (o, number of column indices that were outside the sequence)."""
    B, L, H, d = q.shape
    assert rowptr.dtype == torch.int32 and colidx.dtype == torch.int32 and rowptr.numel() == L + 1
    o = torch.empty_like(q)
    bad = torch.zeros(1, dtype=torch.int32, device=q.device)
    _check(lib.sfb_csr_attention(_stream(), _p(rowptr), _p(colidx), _p(q), _p(k), _p(v), _p(o), dtype_tag(q), B, L, H, d, scale, _p(bad)))
    return o, bad


def bst_sgemm_tn(a, b, lay):
    """C = A^T.B over each block column (bst_sgemm_xn with TN_OP, blocksparse.h:1005-1010): dV = P^T.dO and
    dK = dS^T.Q of the backward pass (transformer_attention_optimize.cu:924,954)."""
    B, L, H, d = _dims(b, lay)
    c = torch.empty_like(b)
    magic, shift = magicu64((d + 63) // 64)
    _check(lib.sfb_bst_sgemm_xn(_stream(), _p(lay.tn_lut), _p(a), _p(b), _p(c), dtype_tag(a), dtype_tag(b), lay.block_size,
                                lay.blocks, B, lay.nb, lay.nb, H, d, lay.heads, lay.nn_lut_dim, TN_OP, magic, shift,
                                lay.tn_max))
    return c


def masked_softmax_grad(dy, y, lay, scale):
    """dx = (dy - sum_row(dy*y)) * y * scale (BlocksparseMaskedSoftmaxGrad<T,V>, blocksparse.h:1164-1227)."""
    assert dy.dtype == y.dtype and dy.shape == y.shape
    B, H = y.shape[:2]
    dx = torch.empty_like(y)
    _check(lib.sfb_masked_softmax_grad(_stream(), _p(lay.nn_lut), _p(dy), _p(y), _p(dx), dtype_tag(y), lay.block_size,
                                       lay.blocks, B, H, lay.nb, lay.heads, lay.nn_lut_dim, lay.nn_max, scale))
    return dx


def rowdot(a, b):
    """sum over the last dimension of a * b, fp32: delta = rowdot(dO, O) for the fused softmax gradient."""
    assert a.shape == b.shape and a.dtype == b.dtype and a.is_contiguous() and b.is_contiguous()
    d = a.shape[-1]
    out = torch.empty(a.shape[:-1], dtype=torch.float32, device=a.device)
    _check(lib.sfb_rowdot(_stream(), _p(out), _p(a), _p(b), a.numel() // d, d, dtype_tag(a)))
    return out


def fused_sddmm_softmax_grad(do, v, p, delta, lay, scale):
    """dS = P * (dO.V^T - delta) * scale in one launch (16-bit operands, 64x64 blocks, 64-wide heads)."""
    B, L, H, d = _dims(do, lay)
    assert p.dtype == do.dtype == v.dtype and delta.dtype == torch.float32 and tuple(delta.shape) == (B, L, H)
    ds = torch.empty_like(p)
    _check(lib.sfb_fused_sddmm_softmax_grad(_stream(), _p(lay.nt_lut), _p(do), _p(v), _p(p), _p(delta), _p(ds), dtype_tag(p),
                                            lay.block_size, lay.blocks, B, lay.nb, H, d, lay.heads, lay.nt_lut_dim, scale))
    return ds


def attention_backward_fused(q, k, v, p, o, do, lay, scale):
    """The backward with the dP / dS pair fused: dV = P^T.dO, dS = P*(dO.V^T - rowdot(dO, O))*scale, dK = dS^T.Q, dQ = dS.K.
    16-bit operands; o is the forward output.  Returns (dq, dk, dv)."""
    dv = bst_sgemm_tn(p, do, lay)
    ds = fused_sddmm_softmax_grad(do, v, p, rowdot(do, o), lay, scale)
    dk = bst_sgemm_tn(ds, q, lay)
    dq = bst_sgemm_xn(ds, k, lay)
    return dq, dk, dv


def attention_backward(q, k, v, p, do, lay, scale, s_dtype=torch.bfloat16):
    """The reference's backward sequence (transformer_attention_optimize.cu:924-964) from the saved probabilities:
    dV = P^T.dO, dP = dO.V^T, dS = softmax_grad(dP, P), dK = dS^T.Q, dQ = dS.K.  Returns (dq, dk, dv)."""
    dv = bst_sgemm_tn(p, do, lay)
    dp = bst_sgemm_nt(do, v, lay, s_dtype)
    ds = masked_softmax_grad(dp, p.to(s_dtype) if p.dtype != s_dtype else p, lay, scale)
    dk = bst_sgemm_tn(ds, q, lay)
    dq = bst_sgemm_xn(ds, k, lay)
    return dq, dk, dv


def fused_sddmm_softmax(q, k, lay, scale, out_dtype=torch.float32, use_mask=False):
    """P = softmax(scale * Q.K^T) in one launch (fusion_attention1/2/_full/_local/2_64,
    fusion_blocksparse.h:400,1212,1636,2030,2456)."""
    B, L, H, d = _dims(q, lay)
    y = torch.empty(B, H, lay.blocks, lay.block_size, lay.block_size, dtype=out_dtype, device=q.device)
    mask = lay.mask_np if use_mask else None
    _check(lib.sfb_fused_sddmm_softmax(_stream(), _p(lay.nn_lut), _p(q), _p(k), _p(mask), _p(y), dtype_tag(q),
                                       _DT[out_dtype], lay.block_size, lay.blocks, B, lay.nb, lay.nb, H, d, lay.heads,
                                       lay.nt_lut_dim, lay.heads, scale))
    return y


def fused_attention(q, k, v, lay, scale=None, use_mask=False, out=None):
    """O = softmax(scale * Q.K^T on the kept blocks).V in one launch (fusion_attention,
    fusion_blocksparse.h:2990-3050)."""
    B, L, H, d = _dims(q, lay)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    o = torch.empty_like(q) if out is None else out
    mask = lay.mask_np if use_mask else None
    _check(lib.sfb_fused_attention(_stream(), _p(lay.nn_lut), _p(q), _p(k), _p(v), _p(o), _p(mask), dtype_tag(q),
                                   lay.block_size, lay.blocks, B, lay.nb, H, d, lay.heads, lay.nt_lut_dim, lay.heads,
                                   scale, lay.nn_max))
    return o


def _row_pitch(t):
    """Row pitch (elements) of a [B, L, H, d] view whose heads are a slice of a wider tensor: rows of one batch element
    and batch elements themselves must follow each other at that pitch."""
    B, L, H, d = t.shape
    sb, sl, sh, sd = t.stride()
    assert sd == 1 and sh == d and sl >= H * d and (B == 1 or sb == L * sl), "not a head slice of a [B, L, H_total, d] tensor"
    return sl


def fused_attention_slice(q, k, v, lay, scale=None, use_mask=False, out=None):
    """fused_attention on views that select some heads (and batch elements) of wider [B, L, H_total, d] tensors, in
    place (sfb_fused_attention_slice): what one rank of a multi-GPU run calls on its share of the (batch, head) pairs."""
    B, L, H, d = _dims(q, lay)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    o = torch.empty(B, L, H, d, dtype=q.dtype, device=q.device) if out is None else out
    pin = _row_pitch(q)
    assert _row_pitch(k) == pin and _row_pitch(v) == pin
    mask = lay.mask_np if use_mask else None
    _check(lib.sfb_fused_attention_slice(_stream(), _p(lay.nn_lut), _p(q), _p(k), _p(v), _p(o), _p(mask), dtype_tag(q),
                                         lay.block_size, lay.blocks, B, lay.nb, H, d, lay.heads, lay.nt_lut_dim, lay.heads,
                                         scale, lay.nn_max, pin, _row_pitch(o)))
    return o


def bias_residual_layernorm(x, bias, resid, gain, beta, want_sum=False, out=None):
    """LayerNorm(resid + (x + bias)) (tensor_add_vector_gpu + tensor_add_tensor_gpu + layernorm_gpu,
    cuda_kernels.h:459,449,334).  Returns (out, sum or None, mean, rstd); out may be x or resid."""
    m, hidden = x.shape
    out = torch.empty_like(x) if out is None else out
    summed = torch.empty_like(x) if want_sum else None
    mean = torch.empty(m, dtype=torch.float32, device=x.device)
    rstd = torch.empty(m, dtype=torch.float32, device=x.device)
    _check(lib.sfb_bias_residual_layernorm(_stream(), _p(out), _p(summed), _p(mean), _p(rstd), _p(x), _p(bias), _p(resid),
                                           _p(gain), _p(beta), m, hidden, dtype_tag(x)))
    return out, summed, mean, rstd


def bias_gelu(x, bias, out=None):
    """(x + bias) * sigmoid(1.702 (x + bias)) (tensor_add_vector_gpu_2048 + gelu_gpu_v2, cuda_kernels.h:471,561)."""
    m, n = x.shape
    out = torch.empty_like(x) if out is None else out
    _check(lib.sfb_bias_gelu(_stream(), _p(out), _p(x), _p(bias), m, n, dtype_tag(x)))
    return out


class HostPipeline:
    """Fused attention on operands that live in pinned HOST memory: the batch is cut into chunks and the
    host->device copies, the kernel and the device->host copy of consecutive chunks overlap on three streams
    (PCIe is full duplex, and the kernel is much shorter than either copy).  Device staging buffers are
    allocated once, here; a call allocates nothing."""

    def __init__(self, shape, dtype, lay, chunks=None, device="cuda"):
        B = shape[0]
        self.chunks = chunks or B
        assert B % self.chunks == 0
        self.lay = lay
        self.q, self.k, self.v, self.o = (torch.empty(shape, dtype=dtype, device=device) for _ in range(4))
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=device) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(self.chunks)]
        self.ev_run = [torch.cuda.Event() for _ in range(self.chunks)]

    def __call__(self, hq, hk, hv, ho, scale):
        B = hq.shape[0]
        per = B // self.chunks
        cur = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        for c in range(self.chunks):
            sl = slice(c * per, (c + 1) * per)
            with torch.cuda.stream(self.s_in):
                self.q[sl].copy_(hq[sl], non_blocking=True)
                self.k[sl].copy_(hk[sl], non_blocking=True)
                self.v[sl].copy_(hv[sl], non_blocking=True)
                self.ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[c])
                fused_attention(self.q[sl], self.k[sl], self.v[sl], self.lay, scale, out=self.o[sl])
                self.ev_run[c].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[c])
                ho[sl].copy_(self.o[sl], non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.s_out)
        cur.wait_event(done)
        return ho
