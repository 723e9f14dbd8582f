"""FlashInternImage backbone + classification head: the caller of the DCNv4 hot path.

A restatement of classification/models/flash_intern_image.py (StemLayer :235-272,
DownsampleLayer :276-304, MLPLayer :308-341, InternImageLayer :344-437, InternImageBlock
:440-537, FlashInternImage :540-770) for the T/S/B/L classification models, without the timm
dependency and without the InternImage-H/G extras (clip projector, level-2 post norms,
residual post norms).  Module and parameter names follow the reference, so its released
`.pth` state dicts load with `load_state_dict`.

Layout: activations stay channels-last.  The stem and downsample convolutions see NHWC
storage through `permute` views in `torch.channels_last` memory format (no transposition
copies), and the tokens handed to `DCNv4` are the same storage viewed as (N, H*W, C).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn
from torch.utils import checkpoint

from . import ops
from .modules import DCNv4


class _ToChannelsFirst(nn.Module):
    def forward(self, x):
        return x.permute(0, 3, 1, 2)


class _ToChannelsLast(nn.Module):
    def forward(self, x):
        return x.permute(0, 2, 3, 1)


class LayerNorm(nn.LayerNorm):
    """torch.nn.LayerNorm (same parameters, same state-dict keys) whose inference forward on CUDA
    runs the library's channels-last kernel: the model normalises millions of rows of 64-512
    channels, which the stock kernel handles one thread block per row.  Whenever autograd needs
    the operation (training) or the kernel does not cover the input, the stock path runs."""

    use_library_kernel = True   # class-wide switch (benchmarks turn it off to time the stock path)

    def forward(self, x):
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)
        if (self.use_library_kernel and not needs_grad and self.elementwise_affine and self.bias is not None
                and len(self.normalized_shape) == 1 and not torch.is_autocast_enabled()
                and ops.layer_norm_supported(x, self.weight)):
            return ops.layer_norm_forward(x, self.weight, self.bias, self.eps)
        return super().forward(x)


def build_norm_layer(dim: int, norm_layer: str, in_format="channels_last", out_format="channels_last",
                     eps: float = 1e-6) -> nn.Sequential:
    """BN works channels-first, LN channels-last; format adapters are parameter-free members of
    the Sequential so that parameter indices match the reference (flash_intern_image.py:34-56)."""
    layers: List[nn.Module] = []
    if norm_layer == "BN":
        if in_format == "channels_last":
            layers.append(_ToChannelsFirst())
        layers.append(nn.BatchNorm2d(dim))
        if out_format == "channels_last":
            layers.append(_ToChannelsLast())
    elif norm_layer == "LN":
        if in_format == "channels_first":
            layers.append(_ToChannelsLast())
        layers.append(LayerNorm(dim, eps=eps))
        if out_format == "channels_first":
            layers.append(_ToChannelsFirst())
    else:
        raise NotImplementedError(f"build_norm_layer does not support {norm_layer}")
    return nn.Sequential(*layers)


def build_act_layer(act_layer: str) -> nn.Module:
    if act_layer == "ReLU":
        return nn.ReLU(inplace=True)
    if act_layer == "SiLU":
        return nn.SiLU(inplace=True)
    if act_layer == "GELU":
        return nn.GELU()
    raise NotImplementedError(f"build_act_layer does not support {act_layer}")


class DropPath(nn.Module):
    """Stochastic depth per sample (the reference takes it from timm)."""

    def __init__(self, drop_prob: float = 0.0):
        super().__init__()
        self.drop_prob = float(drop_prob)

    def forward(self, x):
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1.0 - self.drop_prob
        mask = x.new_empty((x.shape[0],) + (1,) * (x.dim() - 1)).bernoulli_(keep)
        return x * mask / keep


class StemLayer(nn.Module):
    """Two stride-2 3x3 convolutions: (N,3,H,W) -> (N,H/4,W/4,C) channels-last
    (classification/models/flash_intern_image.py:235-272).  FlashInternImage builds it with the
    network's norm layer, LayerNorm (:615-618), so each convolution is followed by a LayerNorm over
    its channels, the first one also by a GELU."""

    def __init__(self, in_chans=3, out_chans=96, act_layer="GELU", norm_layer="BN"):
        super().__init__()
        self.conv1 = nn.Conv2d(in_chans, out_chans // 2, kernel_size=3, stride=2, padding=1)
        self.norm1 = build_norm_layer(out_chans // 2, norm_layer, "channels_first", "channels_first")
        self.act = build_act_layer(act_layer)
        self.conv2 = nn.Conv2d(out_chans // 2, out_chans, kernel_size=3, stride=2, padding=1)
        self.norm2 = build_norm_layer(out_chans, norm_layer, "channels_first", "channels_last")

    def _fused_norm_act(self, x):
        """LayerNorm + GELU over the channels of a channels-last activation in one pass (inference):
        the convolution's (N,C,H,W) result in channels_last memory is the contiguous (N,H,W,C) tensor
        the kernel wants, and so is its input view for the next convolution."""
        ln = self.norm1[1] if len(self.norm1) == 3 and isinstance(self.norm1[1], LayerNorm) else None
        if (ln is None or not isinstance(self.act, nn.GELU) or self.act.approximate != "none"
                or torch.is_grad_enabled() and (x.requires_grad or ln.weight.requires_grad)
                or torch.is_autocast_enabled() or not LayerNorm.use_library_kernel):
            return None
        t = x.permute(0, 2, 3, 1)
        if not (t.is_contiguous() and ops.layer_norm_supported(t, ln.weight)):
            return None
        return ops.layer_norm_forward(t, ln.weight, ln.bias, ln.eps, "gelu").permute(0, 3, 1, 2)

    def forward(self, x):
        x = x.contiguous(memory_format=torch.channels_last)
        if (isinstance(self.norm1[0], nn.Identity) and isinstance(self.norm2[0], nn.Identity)
                and isinstance(self.act, nn.GELU) and self.act.approximate == "none"):
            # BatchNorm stem with the norms folded (fold_batchnorm_): their shift is the convolution
            # bias, applied together with the GELU by one pass over the convolution's output
            x = ops.conv2d_bias_act(x, self.conv1, "gelu")
            return self.norm2(ops.conv2d_bias_act(x, self.conv2, "none")).contiguous()
        x = self.conv1(x)
        fused = self._fused_norm_act(x)
        x = fused if fused is not None else self.act(self.norm1(x))
        return self.norm2(self.conv2(x)).contiguous()


class DownsampleLayer(nn.Module):
    """Stride-2 3x3 convolution doubling the channels, on (N, H*W, C) tokens."""

    def __init__(self, channels, norm_layer="LN"):
        super().__init__()
        self.conv = nn.Conv2d(channels, 2 * channels, kernel_size=3, stride=2, padding=1, bias=False)
        self.norm = build_norm_layer(2 * channels, norm_layer, "channels_first", "channels_first")

    def forward(self, x, shape: Tuple[int, int]):
        H, W = shape
        N, _, C = x.shape
        x = self.conv(x.view(N, H, W, C).permute(0, 3, 1, 2))   # NHWC storage seen as channels_last NCHW
        x = self.norm(x)
        H, W = x.size(2), x.size(3)
        return x.permute(0, 2, 3, 1).reshape(N, H * W, 2 * C), (H, W)


def _single_layer_norm(module) -> Optional[nn.LayerNorm]:
    """The nn.LayerNorm inside a channels-last norm layer built by build_norm_layer, if that is
    all the layer consists of."""
    if isinstance(module, nn.LayerNorm):
        return module
    if isinstance(module, nn.Sequential) and len(module) == 1 and isinstance(module[0], nn.LayerNorm):
        return module[0]
    return None


class _ConvAsLinear:
    """A 1x1 nn.Conv2d seen as the nn.Linear it is (what ops.linear_module_forward reads)."""

    def __init__(self, conv: nn.Conv2d):
        self.weight = conv.weight.view(conv.out_channels, conv.in_channels)
        self.bias = conv.bias
        self.in_features, self.out_features = conv.in_channels, conv.out_channels


class MLPLayer(nn.Module):
    def __init__(self, in_features, hidden_features=None, out_features=None, act_layer="GELU",
                 mlp_fc2_bias=False, drop=0.0):
        super().__init__()
        out_features = out_features or in_features
        hidden_features = hidden_features or in_features
        self.fc1 = nn.Linear(in_features, hidden_features, bias=True)
        self.act = build_act_layer(act_layer)
        self.fc2 = nn.Linear(hidden_features, out_features, bias=mlp_fc2_bias)
        self.drop = nn.Dropout(drop)

    def forward(self, x, shape=None, residual=None, norm=None):
        """fc2(act(fc1(x))) [+ residual], and with `norm` (an nn.LayerNorm) the pair
        (result, norm(result)); at inference GELU, the residual addition and the LayerNorm are
        fused into the two matrix products (dropout is the identity there)."""
        if isinstance(self.act, nn.GELU) and self.act.approximate == "none" and not (self.training and self.drop.p > 0):
            h = ops.linear_module_forward(x, self.fc1, None, "gelu")
            return ops.linear_module_forward(h, self.fc2, residual, "none", norm)
        y = self.drop(self.fc2(self.drop(self.act(self.fc1(x)))))
        y = y if residual is None else residual + y
        return y if norm is None else (y, norm(y))


class InternImageLayer(nn.Module):
    """x + dcn(norm1(x)); x + mlp(norm2(x)) -- or the post-norm / layer-scale variants."""

    def __init__(self, core_op, channels, groups, mlp_ratio=4.0, drop=0.0, drop_path=0.0, act_layer="GELU",
                 norm_layer="LN", post_norm=False, layer_scale=None, offset_scale=1.0, with_cp=False,
                 dcn_output_bias=False, mlp_fc2_bias=False, dw_kernel_size=None):
        super().__init__()
        self.channels, self.groups, self.mlp_ratio, self.with_cp = channels, groups, mlp_ratio, with_cp
        self.norm1 = build_norm_layer(channels, "LN")
        self.post_norm = post_norm
        self.dcn = core_op(channels=channels, group=groups, offset_scale=offset_scale,
                           dw_kernel_size=dw_kernel_size, output_bias=dcn_output_bias)
        self.drop_path = DropPath(drop_path) if drop_path > 0.0 else nn.Identity()
        self.norm2 = build_norm_layer(channels, "LN")
        self.mlp = MLPLayer(in_features=channels, hidden_features=int(channels * mlp_ratio),
                            act_layer=act_layer, drop=drop, mlp_fc2_bias=mlp_fc2_bias)
        self.layer_scale = layer_scale is not None
        if self.layer_scale:
            self.gamma1 = nn.Parameter(layer_scale * torch.ones(channels), requires_grad=True)
            self.gamma2 = nn.Parameter(layer_scale * torch.ones(channels), requires_grad=True)

    def _inner(self, x, shape):
        if self.post_norm:
            a = self.norm1(self.dcn(x, shape))
            x = x + self.drop_path(self.gamma1 * a if self.layer_scale else a)
            m = self.norm2(self.mlp(x, shape))
            x = x + self.drop_path(self.gamma2 * m if self.layer_scale else m)
        elif self._plain_residual():
            x = self._chained(x, shape, None, None)[0]
        else:
            a = self.dcn(self.norm1(x), shape)
            x = x + self.drop_path(self.gamma1 * a if self.layer_scale else a)
            m = self.mlp(self.norm2(x), shape)
            x = x + self.drop_path(self.gamma2 * m if self.layer_scale else m)
        return x

    def _plain_residual(self) -> bool:
        """Pre-norm layer whose two branches are added as they are (no layer scale, no active
        stochastic depth): the additions can ride on the output projection and on fc2."""
        return (not self.post_norm and not self.layer_scale
                and (not self.training or isinstance(self.drop_path, nn.Identity)))

    def forward_chained(self, x, shape, normed=None, next_norm=None):
        """The layer for callers that chain layers (InternImageBlock): `normed` is norm1(x) if the
        previous layer already produced it, `next_norm` the LayerNorm that will be applied to
        this layer's result.  Returns (result, next_norm(result) or None).  At inference each
        LayerNorm is computed in the epilogue of the matrix product that precedes it."""
        if not self._plain_residual() or (self.with_cp and x.requires_grad):
            x = self.forward(x, shape)
            return x, (None if next_norm is None else next_norm(x))
        return self._chained(x, shape, normed, next_norm)

    def _chained(self, x, shape, normed, next_norm):
        n2 = _single_layer_norm(self.norm2)
        a_in = normed if normed is not None else self.norm1(x)
        if n2 is not None:
            x, m_in = self.dcn(a_in, shape, residual=x, norm=n2)
        else:
            x = self.dcn(a_in, shape, residual=x)
            m_in = self.norm2(x)
        nn_ = _single_layer_norm(next_norm) if next_norm is not None else None
        if nn_ is not None:
            x, nxt = self.mlp(m_in, shape, residual=x, norm=nn_)
            return x, nxt
        x = self.mlp(m_in, shape, residual=x)
        return x, (None if next_norm is None else next_norm(x))

    def forward(self, x, shape):
        if self.with_cp and x.requires_grad:
            return checkpoint.checkpoint(self._inner, x, shape, use_reentrant=False)
        return self._inner(x, shape)


class InternImageBlock(nn.Module):
    """`depth` layers at one resolution, a final LayerNorm (pre-norm models) and the downsample."""

    def __init__(self, core_op, channels, depth, groups, downsample=True, mlp_ratio=4.0, drop=0.0,
                 drop_path=0.0, act_layer="GELU", norm_layer="LN", post_norm=False, offset_scale=0.5,
                 layer_scale=None, with_cp=False, dcn_output_bias=False, mlp_fc2_bias=False,
                 dw_kernel_size=None):
        super().__init__()
        self.channels, self.depth, self.post_norm = channels, depth, post_norm
        self.blocks = nn.ModuleList([
            InternImageLayer(core_op=core_op, channels=channels, groups=groups, mlp_ratio=mlp_ratio, drop=drop,
                             drop_path=drop_path[i] if isinstance(drop_path, (list, tuple)) else drop_path,
                             act_layer=act_layer, norm_layer=norm_layer, post_norm=post_norm,
                             layer_scale=layer_scale, offset_scale=offset_scale, with_cp=with_cp,
                             dcn_output_bias=dcn_output_bias, mlp_fc2_bias=mlp_fc2_bias,
                             dw_kernel_size=dw_kernel_size)
            for i in range(depth)])
        if not self.post_norm:
            self.norm = build_norm_layer(channels, "LN")
        self.downsample = DownsampleLayer(channels=channels, norm_layer=norm_layer) if downsample else None

    def forward(self, x, shape):
        normed = None  # norm1 of the next layer (or the level's final norm) applied to x, if already known
        for i, blk in enumerate(self.blocks):
            nxt = self.blocks[i + 1].norm1 if i + 1 < len(self.blocks) else (None if self.post_norm else self.norm)
            x, normed = blk.forward_chained(x, shape, normed, nxt)
        if not self.post_norm:
            x = normed if normed is not None else self.norm(x)
        if self.downsample is not None:
            x, shape = self.downsample(x, shape)
        return x, shape


class FlashInternImage(nn.Module):
    """FlashInternImage-T/S/B/L classifier.  Defaults are the reference constructor's
    (flash_intern_image.py:575-600); `CONFIGS` holds the released model settings."""

    def __init__(self, core_op="DCNv4", channels=64, depths: Sequence[int] = (3, 4, 18, 5),
                 groups: Sequence[int] = (3, 6, 12, 24), num_classes=1000, mlp_ratio=4.0, drop_rate=0.0,
                 drop_path_rate=0.2, drop_path_type="linear", act_layer="GELU", norm_layer="LN",
                 layer_scale=None, offset_scale=0.5, post_norm=False, cls_scale=1.5, with_cp=False,
                 mlp_fc2_bias=False, dcn_output_bias=False, dw_kernel_size=None, **kwargs):
        super().__init__()
        if core_op != "DCNv4":
            raise ValueError("this package provides the DCNv4 core operator only")
        self.core_op, self.num_classes, self.depths = core_op, num_classes, list(depths)
        self.num_levels = len(depths)
        self.channels = channels
        self.num_features = int(channels * 2 ** (self.num_levels - 1))
        self.patch_embed = StemLayer(in_chans=3, out_chans=channels, act_layer=act_layer, norm_layer=norm_layer)
        self.pos_drop = nn.Dropout(p=drop_rate)
        total = sum(depths)
        dpr = [drop_path_rate * i / max(total - 1, 1) for i in range(total)]
        if drop_path_type == "uniform":
            dpr = [drop_path_rate] * total
        self.levels = nn.ModuleList()
        for i in range(self.num_levels):
            self.levels.append(InternImageBlock(
                core_op=DCNv4, channels=int(channels * 2 ** i), depth=depths[i], groups=groups[i],
                mlp_ratio=mlp_ratio, drop=drop_rate, drop_path=dpr[sum(depths[:i]): sum(depths[:i + 1])],
                act_layer=act_layer, norm_layer=norm_layer, post_norm=post_norm,
                downsample=(i < self.num_levels - 1), layer_scale=layer_scale, offset_scale=offset_scale,
                with_cp=with_cp, mlp_fc2_bias=mlp_fc2_bias, dcn_output_bias=dcn_output_bias,
                dw_kernel_size=dw_kernel_size))
        head_dim = int(self.num_features * cls_scale)
        self.conv_head = nn.Sequential(
            nn.Conv2d(self.num_features, head_dim, kernel_size=1, bias=False),
            build_norm_layer(head_dim, "BN", "channels_first", "channels_first"),
            build_act_layer(act_layer))
        self.head = nn.Linear(head_dim, num_classes) if num_classes > 0 else nn.Identity()
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.apply(self._init_weights)
        for m in self.modules():
            if isinstance(m, DCNv4):
                m._reset_parameters()

    @staticmethod
    def _init_weights(m):
        if isinstance(m, nn.Linear):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)
        elif isinstance(m, nn.LayerNorm):  # includes the LayerNorm subclass above
            nn.init.constant_(m.bias, 0)
            nn.init.constant_(m.weight, 1.0)

    def forward_features(self, x):
        x = self.patch_embed(x)                    # (N, H/4, W/4, C) channels-last
        N, H, W, C = x.shape
        x = self.pos_drop(x.view(N, H * W, C))
        shape = (H, W)
        for level in self.levels:
            x, shape = level(x, shape)
        h, w = shape
        conv, act = self.conv_head[0], self.conv_head[2]
        if (isinstance(self.conv_head[1][0], nn.Identity) and conv.bias is not None and conv.kernel_size == (1, 1)
                and conv.stride == (1, 1) and conv.groups == 1 and isinstance(act, nn.GELU)
                and act.approximate == "none"):
            # BatchNorm folded (fold_batchnorm_): the 1x1 head convolution is a Linear over the
            # channels-last tokens, with its bias and the GELU in the same kernel
            y = ops.linear_module_forward(x.reshape(N * h * w, -1), _ConvAsLinear(conv), None, "gelu")
            x = y.view(N, h, w, -1).permute(0, 3, 1, 2)
        else:
            x = self.conv_head(x.view(N, h, w, -1).permute(0, 3, 1, 2))
        return torch.flatten(self.avgpool(x), 1)

    def forward(self, x):
        return self.head(self.forward_features(x))


@torch.no_grad()
def fold_batchnorm_(model: "FlashInternImage") -> "FlashInternImage":
    """Inference-only rewrite, in place: fold every BatchNorm2d of the network into the convolution
    in front of it, using the running statistics, and replace it by an identity.  FlashInternImage
    has one, behind the 1x1 convolution of the classification head (its stem and downsample norms
    are LayerNorms); a stem built with norm_layer='BN' is folded as well.  The model must be in eval
    mode and is no longer trainable (nor state-dict compatible) afterwards."""
    if model.training:
        raise RuntimeError("fold_batchnorm_ is for eval-mode models")

    def fold(conv: nn.Conv2d, bn: nn.BatchNorm2d):
        scale = bn.weight / torch.sqrt(bn.running_var + bn.eps)
        conv.weight.mul_(scale.view(-1, 1, 1, 1).to(conv.weight.dtype))
        bias = conv.bias if conv.bias is not None else torch.zeros_like(bn.running_mean)
        new_bias = (bias.float() - bn.running_mean.float()) * scale.float() + bn.bias.float()
        conv.bias = nn.Parameter(new_bias.to(conv.weight.dtype), requires_grad=False)

    stem = model.patch_embed
    if isinstance(stem.norm1[0], nn.BatchNorm2d) and isinstance(stem.norm2[0], nn.BatchNorm2d):
        fold(stem.conv1, stem.norm1[0])
        stem.norm1[0] = nn.Identity()
        fold(stem.conv2, stem.norm2[0])
        stem.norm2[0] = nn.Identity()
    fold(model.conv_head[0], model.conv_head[1][0])
    model.conv_head[1][0] = nn.Identity()
    return model


class GraphedInference:
    """Replay a model's inference forward as one CUDA graph for a fixed input shape.

    A FlashInternImage-T forward is ~600 kernel launches of a few microseconds each; issued one by
    one the host cannot keep a B200 busy.  The forward is captured once (on a side stream, after
    warm-up) and replayed: `graphed(images)` copies the batch into the static input buffer,
    replays, and returns the static output tensor (valid until the next call)."""

    def __init__(self, model: nn.Module, example: torch.Tensor, warmup: int = 3):
        if not example.is_cuda:
            raise RuntimeError("GraphedInference needs a CUDA example input")
        self.model = model.eval()
        # image batches are kept channels-last, the layout the stem wants: the copy into the static
        # buffer then does the layout change and the stem's own conversion disappears from the graph
        self.static_in = (example.clone(memory_format=torch.channels_last) if example.dim() == 4
                          else example.clone())
        side = torch.cuda.Stream(device=example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):   # also triggers the library's once-per-device set-up
                self.model(self.static_in)
        torch.cuda.current_stream(example.device).wait_stream(side)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = self.model(self.static_in)

    def __call__(self, images: torch.Tensor) -> torch.Tensor:
        self.static_in.copy_(images, non_blocking=True)
        self.graph.replay()
        return self.static_out


# Released classification settings (classification/configs/flash_intern_image_{t,s,b}_1k_224.yaml,
# flash_intern_image_l_22kto1k_384.yaml).
CONFIGS = {
    "t": dict(channels=64, depths=(4, 4, 18, 4), groups=(4, 8, 16, 32), offset_scale=1.0, mlp_ratio=4.0,
              drop_path_rate=0.1),
    "s": dict(channels=80, depths=(4, 4, 21, 4), groups=(5, 10, 20, 40), offset_scale=1.0, mlp_ratio=4.0,
              drop_path_rate=0.4, layer_scale=1e-5, post_norm=True, dw_kernel_size=3),
    "b": dict(channels=112, depths=(4, 4, 21, 4), groups=(7, 14, 28, 56), offset_scale=0.5, mlp_ratio=4.0,
              drop_path_rate=0.5, layer_scale=1e-5, post_norm=True, dw_kernel_size=3),
    "l": dict(channels=160, depths=(5, 5, 22, 5), groups=(10, 20, 40, 80), offset_scale=2.0, mlp_ratio=4.0,
              drop_path_rate=0.1, layer_scale=1e-5, post_norm=True, dw_kernel_size=3,
              dcn_output_bias=True, mlp_fc2_bias=True),
}


def flash_intern_image(size: str = "t", **overrides) -> FlashInternImage:
    cfg = dict(CONFIGS[size])
    cfg.update(overrides)
    return FlashInternImage(**cfg)
