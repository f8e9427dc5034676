"""GPU parity of the individual ops, called through the C ABI, against the CPU oracle."""
import ctypes

import pytest
import torch
import torch.nn.functional as F

from tests.gpu_util import O, random_indices, rel_err, strip_col2_of_extra

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def vl():
    from vtpack_b200 import _lib
    from vtpack_b200 import layers
    _lib.lib()
    return _lib, layers


@pytest.mark.parametrize("B,Hr,Wr,splits,extra", [
    (1, 4, 4, [4, 2, 1], 1), (2, 4, 4, [4, 2, 1], 1), (64, 4, 4, [4, 2, 1], 1), (3, 8, 8, [4, 2, 1], 1),
    (5, 4, 4, [2, 1], 1), (4, 4, 4, [4, 2, 1], 0), (2, 4, 4, [4, 2, 1], 2), (300, 4, 4, [4, 2, 1], 1),
])
def test_index_to_patch_bit_exact(vl, B, Hr, Wr, splits, extra):
    _, layers = vl
    idx = random_indices(B, Hr, Wr, len(splits), seed=B * 7 + Hr)
    sp = torch.tensor(splits)
    ref_p, ref_l = O.grained_sample_index_to_patch(idx, sp, max(splits), extra)
    for dt in (torch.int64, torch.int32):
        p, l = layers.grained_sample_index_to_patch(idx.to(DEV, dt), sp, max(splits), extra)
        assert l.device.type == "cpu" and l.dtype == torch.int64
        assert torch.equal(l, ref_l)
        assert p.dtype == torch.int64 and torch.equal(strip_col2_of_extra(p.cpu()), ref_p)
        assert torch.equal(p._vtp_i32.cpu().long(), p.cpu())
        off = p._vtp_offsets.cpu().long()
        assert torch.equal(off[1:] - off[:-1], ref_l) and off[0] == 0


@pytest.mark.parametrize("k", [0, 2])
def test_index_to_patch_extremes(vl, k):
    _, layers = vl
    sp = torch.tensor([4, 2, 1])
    idx = torch.full((3, 4, 4), k)
    ref_p, ref_l = O.grained_sample_index_to_patch(idx, sp, 4, 1)
    p, l = layers.grained_sample_index_to_patch(idx.to(DEV), sp, 4, 1)
    assert torch.equal(l, ref_l) and torch.equal(strip_col2_of_extra(p.cpu()), ref_p)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,G,C", [(2, 16, 192), (3, 16, 384), (2, 32, 64), (1, 16, 768), (2, 8, 8)])
def test_pool_unpool_bit_exact(vl, dtype, B, G, C):
    _, layers = vl
    if dtype == torch.bfloat16 and C % 8:
        pytest.skip("C must be a multiple of 16 bytes")
    sp = torch.tensor([4, 2, 1])
    idx = random_indices(B, G // 4, G // 4, 3, seed=G + C)
    x = O.make_tokens(B, G * G + 1, C, seed=3).to(dtype)
    patches, lens = O.grained_sample_index_to_patch(idx, sp, 4, 1)
    ref = O.grained_sample_compress(x, patches, G, G, 1)
    p_dev, _ = layers.grained_sample_index_to_patch(idx.to(DEV), sp, 4, 1)
    got = layers.grained_sample_compress(x.to(DEV), p_dev, G, G, 1)
    assert got.dtype == dtype and torch.equal(got.cpu(), ref)
    # plain int64 patch list without the cached int32 mirror (the reference's calling convention)
    got2 = layers.grained_sample_compress(x.to(DEV), patches.to(DEV), G, G, 1)
    assert torch.equal(got2.cpu(), ref)

    q = torch.randn(patches.shape[0], C, generator=torch.Generator().manual_seed(9)).to(dtype)
    for add in (True, False):
        ref_o = O.grained_sample_decompress(q, patches, x, G, G, 1, add)
        got_o = layers.grained_sample_decompress(q.to(DEV), p_dev, x.to(DEV), G, G, 1, add)
        assert torch.equal(got_o.cpu(), ref_o)


def test_pool_all_fine_round_trip(vl):
    _, layers = vl
    sp = torch.tensor([4, 2, 1])
    B, G, C = 4, 16, 384
    idx = torch.zeros(B, 4, 4, dtype=torch.int64)
    x = O.make_tokens(B, 257, C, seed=4).to(torch.bfloat16).to(DEV)
    p, l = layers.grained_sample_index_to_patch(idx.to(DEV), sp, 4, 1)
    assert l.tolist() == [257] * B
    comp = layers.grained_sample_compress(x, p, G, G, 1)
    back = layers.grained_sample_decompress(comp, p, torch.zeros_like(x), G, G, 1, True)
    assert torch.equal(back, x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C", [192, 384, 768])
def test_router_gate(vl, dtype, C):
    from vtpack_b200.layers import DynamicRouter
    B, G = 8, 16
    x = O.make_tokens(B, G * G, C, seed=5).to(dtype)
    r = DynamicRouter(C, [4, 2, 1])
    torch.nn.init.trunc_normal_(r.gate.weight, std=0.02, generator=torch.Generator().manual_seed(6))
    ref = O.router_forward(x.float().reshape(B, G, G, C), r.gate.weight.detach(), r.gate.bias.detach(), 4)
    got = r.to(DEV).eval()(x.to(DEV).reshape(B, G, G, C))     # eval mode: the fused gate kernel
    assert got.dtype == torch.float32
    assert torch.allclose(got.cpu(), ref, rtol=1e-4, atol=1e-5)
    top2 = ref.topk(2, -1).values
    sure = (top2[..., 0] - top2[..., 1]) > 1e-5
    assert torch.equal(r.last_indices.cpu().long()[sure], ref.argmax(-1)[sure])


def test_gate_argmax_ties(vl):
    _lib, _ = vl
    logits = torch.tensor([[1., 1., 1.], [0., 2., 2.], [3., 1., 3.], [-1., -2., -0.5]], device=DEV)
    idx = torch.empty(4, dtype=torch.int32, device=DEV)
    _lib.check(_lib.lib().vtp_gate_argmax(logits.data_ptr(), 4, 3, idx.data_ptr(), None))
    assert idx.tolist() == logits.cpu().argmax(-1).tolist() == [0, 1, 0, 2]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("rows,C", [(5, 192), (1000, 384), (33, 768),
                                    # narrow rows (several rows per warp): PVT stages 1 and 2, ragged row counts
                                    (1, 64), (7, 64), (4099, 64), (1001, 128), (3, 32), (514, 96)])
def test_layernorm(vl, dtype, tol, rows, C):
    from vtpack_b200.models.dge.deit_dge import _layernorm
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(rows, C, generator=g) * 3 + 1).to(dtype)
    ln = torch.nn.LayerNorm(C, eps=1e-6)
    ln.weight.data = torch.randn(C, generator=g)
    ln.bias.data = torch.randn(C, generator=g)
    ref = F.layer_norm(x.float(), (C,), ln.weight, ln.bias, 1e-6)
    got = _layernorm(x.to(DEV), ln.to(DEV))
    assert rel_err(got.float(), ref) < tol


def _linear_case(M, N, K, dtype, gelu, res, flags, seed=0):
    from vtpack_b200.models.dge.deit_dge import _linear
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    lin = torch.nn.Linear(K, N)
    lin.weight.data = (torch.randn(N, K, generator=g) * 0.05).to(dtype).float()
    lin.bias.data = torch.randn(N, generator=g)
    r = torch.randn(M, N, generator=g).to(dtype) if res else None
    ref = F.linear(x.float(), lin.weight, lin.bias)
    if gelu:
        ref = F.gelu(ref)
    if res:
        ref = ref + r.float()
    got = _linear(x.to(DEV), lin.to(DEV), residual=None if r is None else r.to(DEV), gelu=gelu, flags=flags)
    return got, ref


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (130, 192, 192), (257, 768, 192), (64, 1000, 384), (300, 384, 1536)])
@pytest.mark.parametrize("gelu,res", [(False, False), (True, False), (False, True)])
def test_linear_fp32(vl, M, N, K, gelu, res):
    got, ref = _linear_case(M, N, K, torch.float32, gelu, res, 0)
    assert rel_err(got, ref) < 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (130, 192, 192), (257, 768, 192), (64, 1000, 384), (300, 384, 1536),
                                   (1024, 1536, 384),
                                   # narrow, short-K Linears (PVT stages 1 and 2): several tiles per CTA, so the
                                   # staging slabs and the held bias slice go round more than once
                                   (148 * 128 * 5 + 77, 64, 64), (148 * 128 * 3, 128, 64), (148 * 128 * 3 + 5, 128, 128)])
@pytest.mark.parametrize("gelu,res", [(False, False), (True, False), (False, True)])
def test_linear_bf16_tensor_cores(vl, M, N, K, gelu, res):
    _lib, _ = vl
    got, ref = _linear_case(M, N, K, torch.bfloat16, gelu, res, 0)
    assert _lib.device_status() == 0
    assert rel_err(got.float(), ref) < 8e-3          # one bf16 rounding of the output
    got_cc, _ = _linear_case(M, N, K, torch.bfloat16, gelu, res, _lib.FLAG_CUDA_CORES)
    assert rel_err(got.float(), got_cc.float()) < 8e-3


def test_linear_device_side_row_count(vl):
    _lib, _ = vl
    M, N, K = 500, 384, 384
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    m_dev = torch.tensor([137], dtype=torch.int32, device=DEV)
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    _lib.check(_lib.lib().vtp_linear(x.data_ptr(), K, w.data_ptr(), None, None, 0, y.data_ptr(), N, 1, M,
                                     m_dev.data_ptr(), N, K, 0, None))
    ref = x[:137].float() @ w.float().t()
    assert rel_err(y[:137].float(), ref) < 8e-3
    assert bool((y[137:] == 7.0).all())


def _attn_case(dtype, B, N, h, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    d = 64
    L = sum(lens)
    q = torch.randn(h, L, d, generator=g).to(dtype)
    k = torch.randn(h, B, N, d, generator=g).to(dtype)
    v = torch.randn(h, B, N, d, generator=g).to(dtype)
    ref = O.batched_sparse_attention_forward(q.float(), k.float(), v.float(), torch.tensor(lens), d ** -0.5)
    return q, k, v, ref


@pytest.mark.parametrize("B,N,h,lens", [(2, 257, 3, [131, 116]), (3, 257, 6, [17, 257, 64]), (2, 1025, 2, [65, 1025]),
                                        (1, 17, 1, [1])])
def test_attention_fp32(vl, B, N, h, lens):
    _, layers = vl
    q, k, v, ref = _attn_case(torch.float32, B, N, h, lens)
    got = layers.batched_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(lens), 64 ** -0.5)
    assert got.shape == ref.shape and rel_err(got, ref) < 1e-5


@pytest.mark.parametrize("B,N,h,lens", [(2, 257, 3, [131, 116]), (3, 257, 6, [17, 257, 64]), (2, 1025, 2, [65, 1025])])
def test_attention_bf16_cuda_cores(vl, B, N, h, lens):
    _lib, layers = vl
    q, k, v, ref = _attn_case(torch.bfloat16, B, N, h, lens)
    got = layers.batched_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(lens), 64 ** -0.5,
                                          flags=_lib.FLAG_CUDA_CORES)
    assert rel_err(got.float(), ref) < 8e-3


@pytest.mark.parametrize("B,N,h,lens", [(2, 257, 3, [131, 116]), (3, 257, 6, [17, 257, 64]), (2, 1025, 2, [65, 1025]),
                                        (1, 17, 1, [1]), (4, 257, 6, [257, 1, 128, 129]), (2, 65, 2, [65, 17])])
def test_attention_bf16_tensor_cores(vl, B, N, h, lens):
    _lib, layers = vl
    q, k, v, ref = _attn_case(torch.bfloat16, B, N, h, lens, seed=B + N)
    got = layers.batched_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(lens), 64 ** -0.5)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_err(got.float(), ref) < 8e-3
    # softmax rows far from uniform: scaled-up queries
    q2 = (q.float() * 6).to(torch.bfloat16)
    ref2 = O.batched_sparse_attention_forward(q2.float(), k.float(), v.float(), torch.tensor(lens), 64 ** -0.5)
    got2 = layers.batched_sparse_attention(q2.to(DEV), k.to(DEV), v.to(DEV), torch.tensor(lens), 64 ** -0.5)
    assert rel_err(got2.float(), ref2) < 1e-2


def test_attention_strided_views(vl):
    """q / k / v as permuted views of Linear outputs, as the model passes them."""
    _, layers = vl
    g = torch.Generator().manual_seed(3)
    B, N, h, d = 2, 257, 3, 64
    lens = [100, 57]
    qflat = torch.randn(sum(lens), h * d, generator=g).to(DEV)
    kv = torch.randn(B, N, 2, h, d, generator=g).to(DEV)
    qv = qflat.reshape(-1, h, d).permute(1, 0, 2)
    kvp = kv.permute(2, 3, 0, 1, 4)
    ref = O.batched_sparse_attention_forward(qv.cpu().contiguous(), kvp[0].cpu().contiguous(),
                                             kvp[1].cpu().contiguous(), torch.tensor(lens), d ** -0.5)
    got = layers.batched_sparse_attention(qv, kvp[0], kvp[1], torch.tensor(lens), d ** -0.5)
    assert rel_err(got, ref) < 1e-5
    assert got.transpose(0, 1).reshape(-1, h * d).is_contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,W,C,ratio", [(2, 8, 8, 64, 2), (3, 16, 8, 128, 4), (1, 32, 32, 64, 8), (2, 4, 4, 320, 2)])
def test_token_im2col_is_a_strided_convolution(vl, dtype, B, H, W, C, ratio):
    """vtp_token_im2col + a matrix product against F.conv2d(kernel = stride = ratio) on the same
    tokens seen as a [B,C,H,W] map (the weight reordered to columns (dy, dx, c_in)); the gather itself
    is checked bit for bit."""
    _lib, _ = vl
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, H * W, C, generator=g).to(dtype).to(DEV)
    cols = torch.empty(B * (H // ratio) * (W // ratio), ratio * ratio * C, dtype=dtype, device=DEV)
    _lib.check(_lib.lib().vtp_token_im2col(ptr(x), dtype_code(dtype), B, H, W, C, ratio, ptr(cols), stream_ptr(x.device)))
    ref = x.reshape(B, H // ratio, ratio, W // ratio, ratio, C).permute(0, 1, 3, 2, 4, 5).reshape(cols.shape)
    assert torch.equal(cols, ref)
    w = torch.randn(C, C, ratio, ratio, generator=g) * 0.05
    conv = F.conv2d(x.float().cpu().permute(0, 2, 1).reshape(B, C, H, W), w, stride=ratio).flatten(2).transpose(1, 2)
    got = cols.float().cpu() @ w.permute(0, 2, 3, 1).reshape(C, -1).t()
    assert rel_err(got.reshape(conv.shape), conv) < 1e-5


@pytest.mark.parametrize("img_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,S,P", [(2, 32, 4), (3, 24, 12), (1, 36, 4), (2, 256, 4)])
def test_small_patch_im2col_plain_and_padded_rows(vl, dtype, img_dtype, B, S, P):
    """Patches that are not multiples of 8 pixels (PVT's 4 x 4 first stage): the rows equal F.unfold's columns
    rounded to the row dtype, bit for bit; with a padded row pitch the first 3*P*P columns are the same and the
    tail is zero even though the buffer was not."""
    _lib, _ = vl
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    g = torch.Generator().manual_seed(5)
    img = torch.randn(B, 3, S, S, generator=g).to(img_dtype).to(DEV)
    KP, G = 3 * P * P, S // P
    ref = F.unfold(img.float(), kernel_size=P, stride=P).transpose(1, 2).reshape(B * G * G, KP).to(dtype)
    cols = torch.empty(B * G * G, KP, dtype=dtype, device=DEV)
    _lib.check(_lib.lib().vtp_patch_im2col(ptr(img), dtype_code(img_dtype), B, S, P, dtype_code(dtype), ptr(cols),
                                           None, None, 0, None, stream_ptr(img.device)))
    assert torch.equal(cols, ref)
    ld = (KP + 63) // 64 * 64 + 8
    padded = torch.full((B * G * G, ld), 7.0, dtype=dtype, device=DEV)
    _lib.check(_lib.lib().vtp_patch_im2col_padded(ptr(img), dtype_code(img_dtype), B, S, P, dtype_code(dtype), ptr(padded),
                                                  ld, stream_ptr(img.device)))
    assert torch.equal(padded[:, :KP], ref)
    assert bool((padded[:, KP:] == 0).all())
    assert _lib.lib().vtp_patch_im2col_padded(ptr(img), dtype_code(img_dtype), B, S, P, dtype_code(dtype), ptr(padded),
                                              KP - 8, stream_ptr(img.device)) == _lib.ERR_SHAPE


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("C", [64, 128, 320, 512])
def test_layernorm_and_position_rows_in_one_pass(vl, dtype, tol, C):
    """vtp_layernorm_add_rows as a stage embedding uses it: LN(y) + position rows, written behind a cls slot;
    against F.layer_norm + the add in fp32.  The cls slots stay untouched."""
    _lib, _ = vl
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    B, HW = 3, 37
    g = torch.Generator().manual_seed(3)
    y = (torch.randn(B * HW, C, generator=g) * 2 + 0.5).to(dtype).to(DEV)
    pos = torch.randn(HW + 1, C, generator=g).to(dtype).to(DEV)
    w, b = torch.randn(C, generator=g).to(DEV), torch.randn(C, generator=g).to(DEV)
    out = torch.full((B, HW + 1, C), 9.0, dtype=dtype, device=DEV)
    _lib.check(_lib.lib().vtp_layernorm_add_rows(ptr(y), dtype_code(dtype), B * HW, C, C, ptr(w), ptr(b), 1e-6, ptr(pos),
                                                 HW, 1, ptr(out), HW, HW + 1, 1, stream_ptr(y.device)))
    ref = F.layer_norm(y.float(), (C,), w, b, 1e-6).reshape(B, HW, C) + pos[1:].float()
    assert rel_err(out[:, 1:].float(), ref) < tol
    assert bool((out[:, 0] == 9.0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rows_position_embedding_and_cls_rows(vl, dtype):
    """vtp_add_rows as the model uses it: tokens + position embedding written behind a cls slot, then
    the cls rows themselves; compared with the same sums done by PyTorch in the same dtype order."""
    _lib, _ = vl
    from vtpack_b200.runtime import dtype_code, ptr, stream_ptr
    B, HW, C = 3, 64, 192
    g = torch.Generator().manual_seed(2)
    y = torch.randn(B * HW, C, generator=g).to(dtype).to(DEV)
    pos = torch.randn(HW + 1, C, generator=g).to(dtype).to(DEV)
    cls = torch.randn(1, C, generator=g).to(dtype).to(DEV)
    out = torch.zeros(B, HW + 1, C, dtype=dtype, device=DEV)
    lib, st = _lib.lib(), stream_ptr(y.device)
    _lib.check(lib.vtp_add_rows(ptr(y), B * HW, ptr(pos), HW, 1, ptr(out), HW, HW + 1, 1, dtype_code(dtype), B * HW, C, st))
    _lib.check(lib.vtp_add_rows(ptr(cls), 1, ptr(pos), 1, 0, ptr(out), 1, HW + 1, 0, dtype_code(dtype), B, C, st))
    ref = torch.cat(((cls.float() + pos[0:1].float()).expand(B, 1, C),
                     y.float().reshape(B, HW, C) + pos[1:].float()[None]), dim=1).to(dtype)
    assert torch.equal(out, ref)


def test_linear_bf16_narrow_reduction_uses_cuda_cores(vl):
    """K = 48 (PVT's 4 x 4 x 3 patch embedding) is not a multiple of the tensor-core kernel's 64-element
    K box: vtp_linear must still answer, through the CUDA-core kernel."""
    _lib, _ = vl
    got, ref = _linear_case(500, 64, 48, torch.bfloat16, False, False, 0)
    assert rel_err(got.float(), ref) < 8e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_patch_rows_outside_the_declared_shape_are_skipped(vl, dtype):
    """A patch row whose image index or coordinates do not fit the declared [B, N] token array is skipped
    and a code is left in the device status word.  The buffers here are allocated for 4 images and the
    calls declare 2, so the bad rows (image 3; a 4x4 patch starting at column 14 of a 16-wide grid) still
    point inside memory this test owns: even a missing guard could not touch anything else."""
    _lib, _ = vl
    lib = _lib.lib()
    B_alloc, B, G, C = 4, 2, 16, 64
    N = G * G + 1
    code = 0 if dtype == torch.float32 else 1
    g = torch.Generator().manual_seed(31)
    x = torch.randn(B_alloc, N, C, generator=g).to(dtype).to(DEV)
    good = [[0, -1, 0, 1], [0, 0, 0, 4], [1, 4, 8, 2], [1, 15, 15, 1]]
    bad = [[3, 0, 0, 4], [1, 0, 14, 4], [1, 14, 0, 4], [0, -2, 0, 1], [-1, 0, 0, 1], [0, 0, 0, 0]]
    rows = torch.tensor(good[:2] + bad[:3] + good[2:] + bad[3:], dtype=torch.int32, device=DEV)
    L = rows.shape[0]
    is_good = torch.tensor([r in good for r in rows.tolist()])
    assert _lib.device_status() == 0
    comp = torch.full((L, C), 7.0, dtype=dtype, device=DEV)
    _lib.check(lib.vtp_pool(x.data_ptr(), code, B, N, C, G, 1, rows.data_ptr(), None, L, comp.data_ptr(), None, None,
                            0.0, None, None, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 64
    ref = O.grained_sample_compress(x[:B].cpu(), rows.cpu().long()[is_good], G, G, 1)
    assert torch.equal(comp.cpu()[is_good], ref)
    assert bool((comp.cpu()[~is_good] == 7.0).all())            # skipped rows were not written
    out = torch.full((B_alloc, N, C), 5.0, dtype=dtype, device=DEV)
    q = torch.randn(L, C, generator=g).to(dtype).to(DEV)
    _lib.check(lib.vtp_unpool_add(q.data_ptr(), None, code, B, N, C, G, 1, rows.data_ptr(), None, L, None,
                                  out.data_ptr(), None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 64
    assert bool((out[B:] == 5.0).all())                          # nothing beyond the declared images
    touched = (out[:B] != 5.0).any(-1).cpu()
    expect = torch.zeros(B, N, dtype=torch.bool)
    expect[0, 0] = True
    expect[0, 1:].view(G, G)[0:4, 0:4] = True
    expect[1, 1:].view(G, G)[4:6, 8:10] = True
    expect[1, 1:].view(G, G)[15, 15] = True
    assert torch.equal(touched, expect)
    # a later tensor-core launch still runs: the bad-index code does not void launches the way a timed-out wait does
    a = torch.randn(256, 64, generator=g).bfloat16().to(DEV)
    w = torch.randn(64, 64, generator=g).bfloat16().to(DEV)
    y = torch.zeros(256, 64, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.vtp_pool(x.data_ptr(), code, B, N, C, G, 1, rows.data_ptr(), None, L, comp.data_ptr(), None, None,
                            0.0, None, None, None))
    _lib.check(lib.vtp_linear(a.data_ptr(), 64, w.data_ptr(), None, None, 0, y.data_ptr(), 64, 1, 256, None, 64, 64,
                              0, None))
    torch.cuda.synchronize()
    assert rel_err(y.float(), a.float() @ w.float().t()) < 1e-2
    assert _lib.device_status() == 64


def test_attention_offsets_beyond_the_buffers_are_clamped(vl):
    """Offsets that claim more packed rows than q / out hold (offsets[B] > l_max): the rows that exist are
    computed, nothing at or beyond l_max is written, and the status word carries the bad-index code.  The
    out buffer is allocated larger than declared so the check itself stays inside owned memory."""
    _lib, _ = vl
    lib = _lib.lib()
    B, N, h, d = 2, 65, 2, 64
    C = h * d
    l_max, l_alloc = 40, 128
    g = torch.Generator().manual_seed(41)
    q = torch.randn(l_alloc, C, generator=g).bfloat16().to(DEV)
    kv = torch.randn(B, N, 2 * C, generator=g).bfloat16().to(DEV)
    off = torch.tensor([0, 30, 70], dtype=torch.int32, device=DEV)       # image 1 claims rows 30..69
    for flags in (0, _lib.FLAG_CUDA_CORES):
        out = torch.full((l_alloc, C), 3.0, dtype=torch.bfloat16, device=DEV)
        assert _lib.device_status() == 0
        _lib.check(lib.vtp_sparse_attention(q.data_ptr(), C, d, kv.data_ptr(), kv.data_ptr() + C * 2, N * 2 * C, 2 * C,
                                            d, out.data_ptr(), C, d, 1, B, N, h, d, off.data_ptr(), l_max, 64,
                                            d ** -0.5, flags, None))
        torch.cuda.synchronize()
        assert _lib.device_status() == 64
        assert bool((out[l_max:] == 3.0).all())
        k = kv[..., :C].reshape(B, N, h, d).permute(2, 0, 1, 3).float().cpu()
        v = kv[..., C:].reshape(B, N, h, d).permute(2, 0, 1, 3).float().cpu()
        qh = q[:l_max].reshape(l_max, h, d).permute(1, 0, 2).float().cpu()
        ref = O.batched_sparse_attention_forward(qh, k, v, torch.tensor([30, 10]), d ** -0.5)
        got = out[:l_max].reshape(l_max, h, d).permute(1, 0, 2).float().cpu()
        assert rel_err(got, ref) < 2e-2


def test_gelu_epilogue_error_on_a_dense_sweep(vl):
    """The tensor-core Linear evaluates erf-GELU as a tanh fit in packed fp16.  Through an identity weight the
    epilogue sees the inputs themselves: a dense sweep of [-12, 12], the far range up to the fp16 limit, and
    the non-finite values.  Bound: 4e-3 absolute up to |x| = 1 and 4e-3 relative beyond (the fit's 2.7e-4, the
    fp16 arithmetic's 5e-4 rms and one bf16 rounding of the result, 2^-9 relative).  Beyond the fp16 range the
    input saturates at 65504 (the reference would return x itself); -inf gives 0, NaN stays NaN."""
    _lib, _ = vl
    lib = _lib.lib()
    K = 64
    sweep = torch.cat([torch.linspace(-12, 12, 64 * 254), torch.tensor([20., -20., 100., -100., 1000., -1000.,
                       6.0e4, -6.0e4, 0., -0.] + [0.] * 54)]).bfloat16()
    # one non-finite value per row (in a row of the product, inf x 0 from another column would give NaN)
    special = torch.zeros(5, K)
    special[:, 0] = torch.tensor([float("inf"), float("-inf"), float("nan"), 1e5, -1e5])
    special = special.bfloat16().reshape(-1)
    x = torch.cat([sweep, special]).reshape(-1, K)                       # [260, 64]
    M = x.shape[0]
    w = torch.eye(K).bfloat16()
    xd, wd = x.to(DEV), w.to(DEV)
    y = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    _lib.check(lib.vtp_linear(xd.data_ptr(), K, wd.data_ptr(), None, None, 0, y.data_ptr(), K, 1, M, None, K, K,
                              _lib.FLAG_GELU, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    got = y.float().cpu().reshape(-1)
    xin = x.float().reshape(-1)
    n_fin = sweep.numel()
    ref = F.gelu(xin[:n_fin].double()).float()
    err = (got[:n_fin] - ref).abs()
    bound = 4e-3 * xin[:n_fin].abs().clamp_min(1.0)
    assert bool((err <= bound).all()), float((err / bound).max())
    sp = got[n_fin::K][:5]
    assert sp[0] >= 65000 and sp[1] == 0 and torch.isnan(sp[2]) and sp[3] >= 65000 and sp[4] == 0
