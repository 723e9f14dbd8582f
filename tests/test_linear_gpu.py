"""Fused tensor-core Linear (+GELU, +residual) against the unfused PyTorch sequence.

The kernel rounds where the unfused modules round (after the bias, after the activation, after the
residual addition), so the fp32 reference below applies the same roundings and the two may
differ only by the accumulation order of the dot products: one unit in the last place of the
16-bit result.  Tolerances: fp16 rtol 2e-3, bf16 rtol 1.6e-2 (one ulp each)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float16: dict(rtol=2e-3, atol=2e-3), torch.bfloat16: dict(rtol=1.6e-2, atol=1.6e-2)}


def _reference(x, w, b, r, act):
    dt = x.dtype
    y = F.linear(x.float(), w.float(), None if b is None else b.float()).to(dt).float()
    if act == "gelu":
        y = F.gelu(y).to(dt).float()
    if r is not None:
        y = (y + r.float()).to(dt).float()
    return y


# (M, N, K): FlashInternImage projections and MLPs at small batch, ragged row counts, column
# counts that do not fill a tile, one-tile problems and a K that is not a multiple of 64.
SHAPES = [(128, 64, 64), (1, 64, 64), (127, 64, 64), (129, 128, 128), (3136, 256, 64), (3136, 64, 256),
          (784, 512, 128), (784, 128, 512), (196, 1024, 256), (196, 256, 1024), (49, 2048, 512),
          (49, 512, 2048), (1000, 72, 64), (333, 200, 72), (5000, 432, 256), (2, 8, 8), (300, 264, 40)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_variants_match_unfused_sequence(M, N, K, dtype):
    from dcnv4_b200 import ops
    torch.manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).to(dtype)
    b = torch.randn(N, device=DEV).to(dtype)
    r = torch.randn(M, N, device=DEV).to(dtype)
    assert ops.linear_supported(x, w)
    for bias, res, act in [(None, None, "none"), (b, None, "none"), (b, None, "gelu"), (b, r, "none"),
                           (None, r, "gelu")]:
        y = ops.linear_forward(x, w, bias, res, act)
        assert y.shape == (M, N) and y.dtype == dtype
        torch.testing.assert_close(y.float(), _reference(x, w, bias, res, act), **TOL[dtype])
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_gelu_epilogue_is_bit_identical_to_torch_for_every_input(dtype):
    """All 65536 bit patterns pass through an identity weight, so the GELU stage sees each
    one exactly; the result must be torch's erf GELU bit for bit (NaN patterns aside)."""
    from dcnv4_b200 import ops
    bits = torch.arange(65536, dtype=torch.int32, device=DEV).to(torch.int16)
    x = bits.view(dtype).reshape(1024, 64).contiguous()
    x = torch.where(torch.isfinite(x), x, torch.ones_like(x))      # inf/nan would poison whole rows
    x = torch.where(x == 0, torch.zeros_like(x), x)                # -0 + 0 is +0 in any dot product
    y = ops.linear_forward(x, torch.eye(64, device=DEV, dtype=dtype), None, None, "gelu")
    ref = F.gelu(x)
    assert torch.equal(y.view(torch.int16), ref.view(torch.int16))


def test_gelu_epilogue_propagates_non_finite_values():
    from dcnv4_b200 import ops
    x = torch.zeros(128, 64, device=DEV, dtype=torch.float16)
    x[0, 0], x[1, 0], x[2, 0], x[3, 0] = float("inf"), float("-inf"), float("nan"), 60000.0
    w = torch.zeros(64, 64, device=DEV, dtype=torch.float16)
    w[0, 0] = 1.0
    y = ops.linear_forward(x, w, None, None, "gelu")[:, 0]
    ref = F.gelu(x[:, 0])
    assert torch.isinf(y[0]) and y[0] > 0 and torch.isnan(y[1]) and torch.isnan(y[2]) and y[3] == ref[3]
    assert torch.equal(torch.isnan(y), torch.isnan(ref))


def test_output_may_alias_residual_and_batch_dims_are_kept():
    from dcnv4_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(4, 50, 128, device=DEV, dtype=torch.float16)
    w = torch.randn(128, 128, device=DEV, dtype=torch.float16) / 11
    r = torch.randn(4, 50, 128, device=DEV, dtype=torch.float16)
    want = _reference(x.reshape(-1, 128), w, None, r.reshape(-1, 128), "none").reshape(4, 50, 128)
    y = ops.linear_forward(x, w, None, r, "none")
    assert y.shape == (4, 50, 128)
    torch.testing.assert_close(y.float(), want, **TOL[torch.float16])
    # in place: y aliases the residual
    from dcnv4_b200 import _lib
    rc = _lib.lib().dcnv4b200_linear_fwd(x.data_ptr(), w.data_ptr(), None, r.data_ptr(), r.data_ptr(), 1,
                                         200, 128, 128, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.testing.assert_close(r.float(), want, **TOL[torch.float16])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (1, 32, 8), (3136, 64, 256), (1000, 128, 128), (777, 128, 512),
                                   (196, 256, 256), (4099, 256, 1024), (5000, 96, 64), (333, 192, 72)])
def test_linear_with_layernorm_epilogue(M, N, K, dtype):
    """(y, LayerNorm(y)) from one kernel: y must equal the plain fused kernel's bit for bit, and z
    the LayerNorm of that y (fp32 statistics) within one unit in the last place."""
    from dcnv4_b200 import ops
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).to(dtype)
    b = torch.randn(N, device=DEV).to(dtype)
    r = (torch.randn(M, N, device=DEV) * 2 + 1).to(dtype)
    g = (torch.randn(N, device=DEV) * 0.5 + 1).to(dtype)
    beta = torch.randn(N, device=DEV).to(dtype)
    for bias, res in [(b, r), (None, None), (b, None)]:
        y, z = ops.linear_layer_norm_forward(x, w, bias, res, g, beta, 1e-6)
        assert torch.equal(y, ops.linear_forward(x, w, bias, res))
        ref = F.layer_norm(y.float(), (N,), g.float(), beta.float(), 1e-6)
        torch.testing.assert_close(z.float(), ref, **TOL[dtype])
    assert ops.device_status() == 0


def test_layernorm_epilogue_limits_and_module_helper():
    from dcnv4_b200 import _lib, ops
    lib = _lib.lib()
    x = torch.randn(16, 64, device=DEV, dtype=torch.float16)
    st = torch.cuda.current_stream().cuda_stream
    for n, want in ((512, -6), (40, -8), (160, -8)):   # a row must fit one tile; columns in units of 32 / 64
        w = torch.randn(n, 64, device=DEV, dtype=torch.float16)
        y = torch.empty(16, n, device=DEV, dtype=torch.float16)
        g = torch.ones(n, device=DEV, dtype=torch.float16)
        assert lib.dcnv4b200_linear_ln_fwd(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), g.data_ptr(),
                                           g.data_ptr(), 1e-6, y.data_ptr(), 1, 16, n, 64, st) == want
    # the module helper falls back to separate kernels where the fused one does not apply
    lin = torch.nn.Linear(64, 512).to(DEV).half()
    norm = torch.nn.LayerNorm(512, eps=1e-6).to(DEV).half()
    with torch.no_grad():
        y, z = ops.linear_module_forward(x, lin, None, "none", norm)
        torch.testing.assert_close(z, norm(y), **TOL[torch.float16])
        lin2 = torch.nn.Linear(64, 128).to(DEV).half()
        norm2 = torch.nn.LayerNorm(128, eps=1e-6).to(DEV).half()
        y2, z2 = ops.linear_module_forward(x, lin2, None, "none", norm2)      # fused
        torch.testing.assert_close(z2, norm2(y2), **TOL[torch.float16])


def test_linear_rejects_what_it_cannot_do():
    from dcnv4_b200 import _lib, ops
    lib = _lib.lib()
    x = torch.randn(16, 64, device=DEV, dtype=torch.float16)
    w = torch.randn(64, 64, device=DEV, dtype=torch.float16)
    y = torch.empty(16, 64, device=DEV, dtype=torch.float16)
    st = torch.cuda.current_stream().cuda_stream
    call = lambda *a: lib.dcnv4b200_linear_fwd(*a, st)
    assert call(None, w.data_ptr(), None, None, y.data_ptr(), 1, 16, 64, 64, 0) == -1          # null
    assert call(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), 0, 16, 64, 64, 0) == -2   # fp32
    assert call(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), 1, 16, 0, 64, 0) == -3    # shape
    assert call(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), 1, 16, 60, 64, 0) == -8   # N % 8 (channels)
    assert call(x.data_ptr() + 2, w.data_ptr(), None, None, y.data_ptr(), 1, 15, 64, 64, 0) == -4  # alignment
    assert call(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), 1, 16, 64, 64, 7) == -6   # activation (unsupported)
    assert call(x.data_ptr(), w.data_ptr(), None, None, y.data_ptr(), 1, 0, 64, 64, 0) == 0     # empty: no launch
    assert not ops.linear_supported(x.float(), w.float())
    with pytest.raises(ValueError):
        ops.linear_forward(x, w, None, None, "relu")


def test_module_helper_falls_back_when_autograd_needs_it():
    from dcnv4_b200 import ops
    torch.manual_seed(5)
    lin = torch.nn.Linear(64, 256).to(DEV).half()
    x = torch.randn(300, 64, device=DEV, dtype=torch.float16)
    r = torch.randn(300, 256, device=DEV, dtype=torch.float16)
    y_grad = ops.linear_module_forward(x, lin, r, "gelu")       # parameters need grad: stock path
    assert y_grad.requires_grad
    with torch.no_grad():
        y_fused = ops.linear_module_forward(x, lin, r, "gelu")
        ops.FUSED_LINEAR = False
        try:
            y_stock = ops.linear_module_forward(x, lin, r, "gelu")
        finally:
            ops.FUSED_LINEAR = True
    torch.testing.assert_close(y_fused, y_stock, **TOL[torch.float16])
    torch.testing.assert_close(y_fused, y_grad.detach(), **TOL[torch.float16])


def test_flash_intern_image_logits_do_not_depend_on_the_fused_path():
    from dcnv4_b200 import ops
    from dcnv4_b200.flash_intern_image import flash_intern_image
    torch.manual_seed(0)
    model = flash_intern_image("t").to(DEV).half().eval()
    x = torch.randn(4, 3, 224, 224, device=DEV, dtype=torch.float16)
    with torch.no_grad():
        fused = model(x)
        ops.FUSED_LINEAR = False
        try:
            stock = model(x)
        finally:
            ops.FUSED_LINEAR = True
    torch.testing.assert_close(fused.float(), stock.float(), rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("size", ["s", "l"])
def test_post_norm_layer_scale_models_agree_with_the_stock_path(size):
    """FlashInternImage-S / -L: post-norm, layer scale, depthwise offset convolution, channel counts
    (80..640, 160..1280) that are not multiples of 64.  Only fc1+GELU and the plain projections
    are fused there; the logits must not depend on it beyond fp16 rounding."""
    from dcnv4_b200 import ops
    from dcnv4_b200.flash_intern_image import flash_intern_image
    torch.manual_seed(1)
    model = flash_intern_image(size, depths=(1, 1, 2, 1)).to(DEV).half().eval()
    x = torch.randn(2, 3, 96, 128, device=DEV, dtype=torch.float16)
    with torch.no_grad():
        fused = model(x)
        ops.FUSED_LINEAR = False
        try:
            stock = model(x)
        finally:
            ops.FUSED_LINEAR = True
    assert torch.isfinite(fused).all()
    torch.testing.assert_close(fused.float(), stock.float(), rtol=1e-2, atol=2e-3)
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("rows,C", [(1, 8), (1000, 32), (12544, 64), (333, 80), (7, 768), (100000, 32)])
def test_bias_act_matches_the_separate_add_and_gelu(rows, C, dtype):
    from dcnv4_b200 import ops
    torch.manual_seed(rows + C)
    x = (torch.randn(rows, C, device=DEV) * 2).to(dtype)
    b = torch.randn(C, device=DEV).to(dtype)
    for act in ("none", "gelu"):
        want = x + b                                   # rounded to the storage type, as the add_ would
        if act == "gelu":
            want = F.gelu(want)
        got = ops.bias_act_(x.clone(), b, act)
        assert torch.equal(got, want), (act, (got.float() - want.float()).abs().max())
    assert ops.device_status() == 0


def test_folded_stem_uses_bias_act_and_matches_the_stock_path():
    import copy
    from dcnv4_b200 import ops
    from dcnv4_b200.flash_intern_image import flash_intern_image, fold_batchnorm_
    torch.manual_seed(2)
    model = fold_batchnorm_(flash_intern_image("t").to(DEV).half().eval())
    stem = model.patch_embed
    with torch.no_grad():
        stem.conv1.bias.normal_(0, 0.5)
        stem.conv2.bias.normal_(0, 0.5)
        x = torch.randn(3, 3, 64, 96, device=DEV, dtype=torch.float16)
        fused = stem(x)
        ops.FUSED_LINEAR = False
        try:
            stock = stem(x)
        finally:
            ops.FUSED_LINEAR = True
    assert fused.shape == stock.shape == (3, 16, 24, 64)
    torch.testing.assert_close(fused, stock, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("M,K,n1,n2", [(3136, 64, 64, 112), (1000, 128, 128, 216), (196, 256, 256, 432),
                                       (49, 512, 512, 864), (130, 72, 64, 8), (5000, 64, 192, 40)])
def test_two_linears_in_one_product(M, K, n1, n2, dtype):
    """value and offset/mask projections of a DCNv4 layer (FlashInternImage-T stage shapes first):
    each output must equal the single-output kernel's bit for bit."""
    from dcnv4_b200 import ops
    torch.manual_seed(M + K + n1)
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (torch.randn(n1 + n2, K, device=DEV) / K ** 0.5).to(dtype)
    b = torch.randn(n1 + n2, device=DEV).to(dtype)
    for bias in (b, None):
        y1, y2 = ops.linear_pair_forward(x, w, bias, n1)
        assert y1.shape == (M, n1) and y2.shape == (M, n2) and y1.is_contiguous() and y2.is_contiguous()
        assert torch.equal(y1, ops.linear_forward(x, w[:n1].contiguous(), None if bias is None else bias[:n1].contiguous()))
        assert torch.equal(y2, ops.linear_forward(x, w[n1:].contiguous(), None if bias is None else bias[n1:].contiguous()))
    assert ops.device_status() == 0


def test_dcnv4_module_pairs_its_projections_and_tracks_weight_updates():
    from dcnv4_b200 import ops
    from dcnv4_b200.modules.dcnv4 import DCNv4
    torch.manual_seed(4)
    m = DCNv4(channels=64, group=4).to(DEV).half().eval()
    with torch.no_grad():
        m.offset_mask.weight.normal_(0, 0.1)
        m.offset_mask.bias.uniform_(0, 1)
    x = torch.randn(2, 14 * 14, 64, device=DEV, dtype=torch.float16)

    def both():
        with torch.no_grad():
            fused = m(x)
            ops.FUSED_LINEAR = False
            try:
                stock = m(x)
            finally:
                ops.FUSED_LINEAR = True
        return fused, stock

    fused, stock = both()
    torch.testing.assert_close(fused, stock, **TOL[torch.float16])
    assert "_paired_proj" in m.__dict__
    with torch.no_grad():                      # an in-place update must invalidate the stacked copy
        m.value_proj.weight.mul_(0.5)
    fused2, stock2 = both()
    torch.testing.assert_close(fused2, stock2, **TOL[torch.float16])
    assert not torch.allclose(fused2, fused)
