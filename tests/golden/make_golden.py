"""Generate tests/golden/ref_golden.pt by EXECUTING THE REFERENCE'S OWN SOURCE on CPU.

Usage (needs the HyC-LoRA-release checkout; the fixtures it writes are committed,
so the test-suite itself never needs the checkout):

    python tests/golden/make_golden.py /path/to/HyC-LoRA-release

What runs:
  * the reference's pure-PyTorch functions of operators/compress_function.py, imported
    unchanged (statistics, softmax prune / to_dense, update_dict);
  * the reference's Triton kernels (operators/compress_function_kernel.py, the two
    triton_fuse_lora_silu_hadamard_*_kernels.py files, the RMSNorm forward / backward kernels of
    operators/rmsnorm_kernels.py, the softmax backward kernel of operators/softmax_kernels.py and
    the rotary kernel of operators/rope_kernels.py), unchanged, through the Triton CPU
    interpreter.  The kernels are launched through ``.fn`` (the autotuner needs a GPU
    driver) with the tile sizes of their autotune configs.  Two interpreter repairs are
    applied, neither touches kernel source: (1) the interpreter keeps bf16 as raw uint16
    and would do arithmetic on the bits and truncate on down-casts, so bf16 binary ops,
    dots and float conversions are replaced by correct round-to-nearest-even versions;
    (2) the three libdevice calls the kernels use (round, float2uint_rn, uint2float_rn)
    are given their C semantics (roundf = halves away from zero); (3) ``tl.sum`` of a bf16
    tensor accumulates in fp32 and returns fp32, as in the Triton release the reference pins
    (triton==2.3.0, requirements.txt:12: ``sum`` promotes its input with
    ``_promote_reduction_input``); the installed interpreter would add up the raw bit patterns.
"""
import os, sys
os.environ['TRITON_INTERPRET'] = '1'
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('HYC_REFERENCE', '')
assert REF and os.path.isdir(REF), 'pass the path of the HyC-LoRA-release checkout'
sys.path.insert(0, REF)
import numpy as np, torch, triton
import triton.language as tl
import triton.runtime.interpreter as ti

def _bits_to_f32(a16):
    return (a16.astype(np.uint32) << 16).view(np.float32)
def _f32_to_bf16bits(f):
    t = torch.from_numpy(np.ascontiguousarray(f, dtype=np.float32)).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16).reshape(f.shape)

_np_float = {tl.float16: np.float16, tl.float32: np.float32, tl.float64: np.float64}
def _convert_float(input, input_dtype, output_dtype, rounding_mode):
    # correct (round-to-nearest-even) float conversion between fp16/bf16/fp32/fp64
    if input_dtype == tl.bfloat16:
        v = _bits_to_f32(np.asarray(input).view(np.uint16))
    else:
        v = np.asarray(input).view(_np_float[input_dtype])
    if output_dtype == tl.bfloat16:
        return _f32_to_bf16bits(v.astype(np.float32))
    out = v.astype(_np_float[output_dtype])
    return out.view(getattr(np, f"uint{output_dtype.primitive_bitwidth}"))
ti._convert_float = _convert_float

_orig_binary = ti.InterpreterBuilder.binary_op
def binary_op(self, lhs, rhs, op):
    if lhs.dtype.scalar == tl.bfloat16 and rhs.dtype.scalar == tl.bfloat16:
        out = op(_bits_to_f32(lhs.data), _bits_to_f32(rhs.data))
        if out.dtype == np.bool_:
            return ti.TensorHandle(out, tl.int1)
        return ti.TensorHandle(_f32_to_bf16bits(out), tl.bfloat16)
    return _orig_binary(self, lhs, rhs, op)
ti.InterpreterBuilder.binary_op = binary_op
for nm, op in dict(create_fadd=np.add, create_fmul=np.multiply, create_fdiv=np.divide, create_fsub=np.subtract,
                   create_fcmpOLT=np.less, create_fcmpOGT=np.greater, create_fcmpOLE=np.less_equal,
                   create_fcmpOGE=np.greater_equal, create_fcmpOEQ=np.equal).items():
    setattr(ti.InterpreterBuilder, nm, (lambda op: lambda self, l, r: self.binary_op(l, r, op))(op))

_orig_dot = ti.InterpreterBuilder.create_dot
def create_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
    if a.dtype.scalar == tl.bfloat16:
        a = ti.TensorHandle(_bits_to_f32(a.data), tl.float32)
        b = ti.TensorHandle(_bits_to_f32(b.data), tl.float32)
    return _orig_dot(self, a, b, d, input_precision, max_num_imprecise_acc)
ti.InterpreterBuilder.create_dot = create_dot
ti.InterpreterBuilder.get_bf16 = lambda self, v: ti.TensorHandle(_f32_to_bf16bits(np.array([v], dtype=np.float32)), tl.bfloat16)

def _sum_bf16_as_f32(self, input):
    if input.dtype.scalar == tl.bfloat16:
        v = _bits_to_f32(np.asarray(input.handle.data).view(np.uint16))
        return self.to_tensor(np.sum(v, axis=self.axis, keepdims=self.keep_dims, dtype=np.float32), tl.float32)
    return self.to_tensor(np.sum(input.handle.data, axis=self.axis, keepdims=self.keep_dims), input.dtype)
ti.ReduceOps.sum = _sum_bf16_as_f32

class LibdeviceShim:   # semantics of the three libdevice calls the kernels use
    @staticmethod
    def round(x):      # C roundf: halves away from zero; frac is exact in fp32
        t = tl.where(x >= 0, tl.floor(x), tl.ceil(x))
        f = x - t
        return tl.where(f >= 0.5, t + 1.0, tl.where(f <= -0.5, t - 1.0, t))
    float2uint_rn = staticmethod(lambda x: x.to(tl.uint32))   # argument already integral
    uint2float_rn = staticmethod(lambda x: x.to(tl.float32))

import operators.compress_function_kernel as ck
import operators.compress_function as cf
import operators.triton_fuse_lora_silu_hadamard_forward_kernels as fk
import operators.triton_fuse_lora_silu_hadamard_backward_kernels as bk
import operators.rmsnorm_kernels as rk
import operators.softmax_kernels as sk
import operators.rope_kernels as pk
for m in (ck, fk, bk):
    m.tl_math = LibdeviceShim

def _grid(M, N, B): return (triton.cdiv(M, 32) * triton.cdiv(N, 32), B)

def ref_quant(x, s, q, z=None):
    B, M, N = x.shape; epp = 8 // q
    out = torch.empty((B, M, N // epp), dtype=torch.uint8)
    if z is None:
        ck.compression_quantization_kernel.fn[_grid(M, N, B)](x, out, s, B, M, N, *x.stride(), *out.stride(), s.stride(1), q, epp,
            BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, GROUP_SIZE_M=4)
    else:
        z = z.to(torch.bfloat16)
        ck.compression_quantization_with_zero_point_kernel.fn[_grid(M, N, B)](x, out, s, z, B, M, N, *x.stride(), *out.stride(), s.stride(1), z.stride(1), q, epp,
            BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, GROUP_SIZE_M=8)
    return out

def ref_dequant(qt, s, q, z=None):
    B, M, _ = qt.shape; N = s.shape[-1]; epp = 8 // q
    x = torch.empty((B, M, N), dtype=torch.bfloat16)
    if z is None:
        ck.decompression_dequantization_kernel.fn[_grid(M, N, B)](x, qt, s, B, M, N, *x.stride(), *qt.stride(), s.stride(1), q, epp,
            BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, GROUP_SIZE_M=8)
    else:
        z = z.to(torch.bfloat16)
        ck.decompression_dequantization_with_zero_point_kernel.fn[_grid(M, N, B)](x, qt, s, z, B, M, N, *x.stride(), *qt.stride(), s.stride(1), z.stride(1), q, epp,
            BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, GROUP_SIZE_M=8)
    return x

def ref_fused_fwd(xa1, b1, x1, s1, xa2, b2, x2, s2, q):
    B, M, N = x1.shape; R = b1.shape[0]; epp = 8 // q
    q1 = torch.empty((B, M, N // epp), dtype=torch.uint8); q2 = torch.empty_like(q1)
    o = torch.empty((B, M, N), dtype=torch.bfloat16)
    b1 = b1.contiguous(); b2 = b2.contiguous()
    fk.triton_fuse_silu_forward_kernel.fn[_grid(M, N, B)](xa1, b1, x1, q1, s1, xa2, b2, x2, q2, s2, o, B, M, N,
        *xa1.stride(), *b1.stride(), *x1.stride(), *q1.stride(), s1.stride(1), q, epp,
        BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=R, GROUP_SIZE_M=4)
    return q1, q2, o

def ref_fused_bwd(xa1, b1, q1, s1, xa2, b2, q2, s2, g, q):
    B, M, N = g.shape; R = b1.shape[0]; epp = 8 // q
    o = torch.empty((B, M, N), dtype=torch.bfloat16); gg = torch.empty_like(o); gu = torch.empty_like(o)
    bk.triton_fuse_silu_backward_kernel.fn[_grid(M, N, B)](xa1, b1, q1, s1, xa2, b2, q2, s2, g, o, gg, gu, B, M, N,
        *xa1.stride(), *b1.stride(), *g.stride(), *q1.stride(), s1.stride(1), q, epp,
        BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=R, GROUP_SIZE_M=4)
    return o, gg, gu


def ref_rmsnorm_fwd(x, w, eps):
    """The launch of ``rmsnorm_forward`` (operators/rmsnorm_kernels.py:116-150) on CPU tensors (the wrapper itself
    allocates on "cuda")."""
    x = x.contiguous(); y = torch.empty_like(x)
    x_arg = x.reshape(-1, x.shape[-1]); M, N = x_arg.shape
    mean = torch.zeros((M,), dtype=torch.float32); rstd = torch.empty((M,), dtype=torch.float32)
    BLOCK = min(65536 // x.element_size(), triton.next_power_of_2(N))
    rk._rms_norm_fwd_fused[(M,)](x_arg, y, w, mean, rstd, x_arg.stride(0), N, eps, BLOCK_SIZE=BLOCK)
    return y, rstd, BLOCK

def ref_rmsnorm_bwd(dy, x, w, rstd, eps, BLOCK):
    """The launch of ``rmsnorm_backward`` (:153-185).  The interpreter runs the programs one after the other, so the
    lock the kernel spins on (:103-113) is always free."""
    N = w.shape[0]
    G = 64
    if N <= 8192: G = 96
    if N <= 4096: G = 128
    if N <= 1024: G = 256
    locks = torch.zeros(2 * G, dtype=torch.int32); dw = torch.zeros((G, N), dtype=x.dtype)
    dx = torch.empty_like(dy)
    x_arg = x.reshape(-1, x.shape[-1]); M, N = x_arg.shape
    mean = torch.zeros((M,), dtype=torch.float32)
    rk._rms_norm_bwd_dx_fused[(M,)](dx, dy, dw, x, w, mean, rstd, locks, x_arg.stride(0), N, eps,
                                    BLOCK_SIZE_N=BLOCK, GROUP_SIZE_M=G)
    return dx

def ref_softmax_bwd(y, g):
    """``softmax_backward`` (operators/softmax_kernels.py:41-56) is plain host code: called as it is."""
    return sk.softmax_backward(y, g)

def ref_rope(x, cos, sin, backward):
    """``rope_forward`` / ``rope_backward`` (operators/rope_kernels.py:81-131), called as they are."""
    if not backward:
        return pk.rope_forward(x.clone(), cos, sin)
    B, M, n, d = x.shape
    BLOCK, warps = pk.calculate_settings(d // 2)
    div, mod = divmod(n, pk.ROPE_GROUP_SIZE)
    return pk.rope_backward(x.clone(), cos, sin, div + (mod != 0), BLOCK, warps)


def main():
    out = {}
    g = torch.Generator().manual_seed(20240)
    randn = lambda *s: torch.randn(*s, generator=g)
    B, M, N, R = 2, 64, 128, 16
    for q in (2, 4, 8):
        d = {}
        x = randn(B, M, N)
        x[:, :, 5] *= 30; x[:, :, 77] *= 30          # planted outlier channels
        x[0, :, 9] = 0.25                             # a constant column (zero range)
        x = x.to(torch.bfloat16)
        d['x'] = x
        # a-1, a-2, a-3
        s = cf.get_statistics_only_quant(x, q, 'per-channel')
        s_safe = s + (s == 0) * 1e-3
        s_safe = s_safe.to(torch.bfloat16)
        d['scale'] = s; d['scale_safe'] = s_safe
        d['packed'] = ref_quant(x, s_safe, q)
        d['dequant'] = ref_dequant(d['packed'], s_safe, q)
        # a-8 zero-point variant (scale without the zero guard; use a tensor without constant columns)
        xz = randn(B, M, N).to(torch.bfloat16) + 1.5
        xz = xz.to(torch.bfloat16)
        sz, z = cf.get_statistics_only_quant_zero_point(xz, q, 'per-channel')
        d['xz'] = xz; d['zp_scale'] = sz; d['zp'] = z
        d['zp_packed'] = ref_quant(xz, sz, q, z)
        d['zp_dequant'] = ref_dequant(d['zp_packed'], sz, q, z)
        # a-4, a-5, a-6: channel-base path; ratio 2/128 -> k = 2
        ratio = 2.0 / N
        idx, cs = cf.get_statistics_channel_base(x, ratio, q, 'per-channel')
        d['cb_ratio'] = ratio; d['cb_idx'] = idx; d['cb_scale'] = cs
        xc = x.clone()
        x_outlier = xc[:, :, idx]          # compress_function.py:129
        xc[:, :, idx] = 0                  # compress_function.py:130
        d['cb_outlier'] = x_outlier.clone()
        d['cb_packed'] = ref_quant(xc, cs, q)
        xr = ref_dequant(d['cb_packed'], cs, q)
        xr[:, :, idx] = x_outlier          # compress_function.py:169
        d['cb_restored'] = xr
        # 4-D head layout statistics (compress_function.py:46-48)
        xh = randn(B, 4, M, 32).to(torch.bfloat16)
        d['xh'] = xh; d['xh_scale'] = cf.get_statistics_only_quant(xh, q, 'per-channel')
        # a-11, a-12
        xa1 = randn(B, M, R).bfloat16(); xa2 = randn(B, M, R).bfloat16()
        b1 = (randn(R, N) * 0.05).bfloat16(); b2 = (randn(R, N) * 0.05).bfloat16()
        x1 = randn(B, M, N).bfloat16(); x2 = randn(B, M, N).bfloat16()
        s1 = cf.get_statistics_only_quant(x1, q, 'per-channel'); s2 = cf.get_statistics_only_quant(x2, q, 'per-channel')
        q1, q2, o = ref_fused_fwd(xa1, b1, x1, s1, xa2, b2, x2, s2, q)
        go = randn(B, M, N).bfloat16()
        bo, gg, gu = ref_fused_bwd(xa1, b1, q1, s1, xa2, b2, q2, s2, go, q)
        d.update(f_xa1=xa1, f_xa2=xa2, f_b1=b1, f_b2=b2, f_x1=x1, f_x2=x2, f_s1=s1, f_s2=s2,
                 f_q1=q1, f_q2=q2, f_o=o, f_go=go, f_bo=bo, f_ggate=gg, f_gup=gu)
        out[f'q{q}'] = d
    # a-9: attention-map prune (compress_function.py:30-32, 309-317)
    logits = 3 * randn(2, 4, 64, 64)
    logits = logits + torch.triu(torch.full((64, 64), float('-inf')), diagonal=1)
    a = torch.softmax(logits, dim=-1).to(torch.bfloat16)
    thr = cf.get_statistics_softmax(a, 0.05)
    sp = cf.compression_softmax(a, thr)
    thr_mean = (thr * 3 + 0.0123) / 4          # a threshold that is not a bf16 value (post-calibration running mean)
    sp2 = cf.compression_softmax(a, thr_mean)
    out['softmax'] = dict(a=a, ratio=0.05, thr=thr, idx=sp.coalesce().indices().clone(), val=sp.coalesce().values().clone(),
                          dense=cf.decompression_softmax(sp).reshape(a.shape),
                          thr2=thr_mean, idx2=sp2.coalesce().indices().clone(), val2=sp2.coalesce().values().clone())
    # a-14: RMSNorm forward / backward (operators/rmsnorm_kernels.py:10-54, 58-113)
    xs = randn(3, 40, 192); xs[:, :, 7] *= 25
    xs = xs.to(torch.bfloat16)
    wn = (1 + 0.1 * randn(192)).to(torch.bfloat16)
    yn, rstd, BLOCK = ref_rmsnorm_fwd(xs, wn, 1e-5)
    dyn = randn(3, 40, 192).to(torch.bfloat16)
    dxn = ref_rmsnorm_bwd(dyn, xs, wn, rstd, 1e-5, BLOCK)
    out['rmsnorm'] = dict(x=xs, w=wn, eps=1e-5, y=yn, rstd=rstd, dy=dyn, dx=dxn)
    # a-15: softmax backward (operators/softmax_kernels.py:7-38) on a causal map
    ys = a[:, :2].contiguous()
    gs = randn(*ys.shape).to(torch.bfloat16)
    out['softmax_bwd'] = dict(y=ys, g=gs, o=ref_softmax_bwd(ys, gs))
    # rotary embedding (operators/rope_kernels.py:38-78), bf16 and fp32 tables
    pos = torch.arange(24, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))
    emb = torch.cat([torch.outer(pos, inv)] * 2, dim=-1)
    xr_ = randn(2, 20, 6, 64).to(torch.bfloat16)
    rp = dict(x=xr_)
    for nm, dt in (('bf16', torch.bfloat16), ('f32', torch.float32)):
        c, s_ = emb.cos().to(dt), emb.sin().to(dt)
        rp['cos_' + nm] = c; rp['sin_' + nm] = s_
        rp['fwd_' + nm] = ref_rope(xr_, c, s_, False)
        rp['bwd_' + nm] = ref_rope(xr_, c, s_, True)
    out['rope'] = rp
    # a-10: update_dict running mean (compress_function.py:15-27)
    old = {'outlier_channel_index': None, 'scale': None}
    hist = []
    for it in range(3):
        new = {'outlier_channel_index': torch.tensor([it, it + 1]), 'scale': (randn(1, 8).abs() + 0.1).bfloat16()}
        hist.append({k: v.clone() for k, v in new.items()})
        old = cf.update_dict(old, new, it)
    out['update_dict'] = dict(history=hist, final={k: v.clone() for k, v in old.items()})
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'ref_golden.pt')
    torch.save(out, dst)
    print('wrote', dst, os.path.getsize(dst), 'bytes')


if __name__ == '__main__':
    main()
