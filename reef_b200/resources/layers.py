"""Layer-level helpers on top of :class:`Graph`: each call appends one fused kernel.

The fused-op families and their positional argument order are the ones the
reference's TVM build produced (reference: resource/resnet18/resnet18.json,
resource/resnet152/resnet152.cu:315-374,771-841,4390-4474):

=====================================  ==========================================
family                                 args (storage indices, in order)
=====================================  ==========================================
fused_add                              out, in, bias            (NCHW, model input)
fused_add_nn_relu                      out, in, bias            (NHWC)
fused_nn_conv2d                        in, W, out
fused_nn_conv2d_nn_relu                in, W, out
fused_nn_conv2d_add                    in, W, out, residual
fused_nn_conv2d_add_nn_relu            in, W, out, bias
fused_nn_conv2d_add_add_nn_relu        in, W, out, residual, bias
fused_nn_conv2d_add_multiply_add_nn_relu  in, W, out, residual, gamma, beta
fused_nn_max_pool2d[_add_nn_relu]      in, out[, bias]
fused_nn_avg_pool2d                    in, out
fused_nn_global_avg_pool2d             in, out
fused_nn_batch_flatten                 out, in
fused_nn_dense_add[_nn_relu]           x, W, out, bias
fused_nn_softmax                       in, out
=====================================  ==========================================

Synthetic parameters follow the benchmark configs: He-normal conv weights,
BatchNorm (gamma~U(0.5,1.5), beta,mean~N(0,0.1), var~U(0.5,1.5), eps 2e-5)
folded offline into a per-channel scale (absorbed by the adjacent conv weights)
and a bias, exactly the form the reference graphs carry (bias-only
``fused_add_nn_relu`` / ``max_pool2d_add_nn_relu`` ops, reference:
resource/resnet18/resnet18.json kernels 0-2,10).
"""
from __future__ import annotations

import numpy as np

from .graph import Graph, Tensor, kname, tuned_plan

BN_EPS = 2e-5


def round_tf32(a):
    """Round fp32 values to the nearest TF32 (10 explicit mantissa bits), ties away from zero."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    u = (u + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


class Builder:
    def __init__(self, name: str, seed: int, conv_impl: str = "auto"):
        self.g = Graph(name)
        self.seed = int(seed)
        self._n = 0
        self.conv_impl = conv_impl
        # "tc_stem" as conv_impl: also the first convolution goes to the tensor cores (4-channel channels-last
        # input).  Measured slower than the CUDA-core stem (ResNet-152 replay 1.04 -> 1.09 ms): with 4 real
        # channels per 32-channel K block the operand tiles are 7/8 zero fill, so it is not the default.
        self.tc_stem = conv_impl == "tc_stem"
        # the first convolution by default: an im2col gather of the planar input (reef_im2col_nchw) followed by a 1x1
        # tensor-core convolution over the flattened taps; "simt_stem" keeps the reference's planar convolution on CUDA
        # cores for the first layer only (the schedule this one is measured against)
        self.im2col_stem = conv_impl in ("auto", "tc")
        if self.tc_stem or conv_impl == "simt_stem":
            self.conv_impl = "auto"

    # ---- randomness ----------------------------------------------------
    def rng(self) -> np.random.Generator:
        self._n += 1
        return np.random.default_rng([self.seed, self._n])

    def bn(self, c: int):
        """Folded BatchNorm: returns (scale s > 0, shift t) with y = s*x + t."""
        r = self.rng()
        gamma = r.uniform(0.5, 1.5, c)
        beta = r.normal(0.0, 0.1, c)
        mean = r.normal(0.0, 0.1, c)
        var = r.uniform(0.5, 1.5, c)
        s = gamma / np.sqrt(var + BN_EPS)
        t = beta - mean * s
        return s.astype(np.float32), t.astype(np.float32)

    def he_conv(self, co, kh, kw, ci):
        """He-normal weights, OHWI."""
        std = np.sqrt(2.0 / (ci * kh * kw))
        return self.rng().normal(0.0, std, (co, kh, kw, ci)).astype(np.float32)

    # ---- tensors -------------------------------------------------------
    def new_act(self, h, w, c) -> Tensor:
        return Tensor(self.g.temp(h * w * c), h, w, c)

    def slice_of(self, buf: Tensor, coff: int, c: int) -> Tensor:
        return Tensor(buf.idx, buf.h, buf.w, c, buf.cstride, buf.coff + coff)

    # ---- ops -----------------------------------------------------------
    def input_bias_nchw(self, data_idx: int, c: int, h: int, w: int, bias) -> Tensor:
        out = Tensor(self.g.temp(c * h * w), h, w, c)
        b = self.g.param(bias)
        self.g.kernel(kname("fused_add", c=c, hw=h * w), [out.idx, data_idx, b])
        return out

    def input_nhwc4(self, data_idx: int, c: int, h: int, w: int, bias=None) -> Tensor:
        """The planar model input (+ per-channel bias) as a channels-last tensor with 4 channels per pixel, the
        layout the tensor-core convolution can read (the 4th channel is zero)."""
        out = Tensor(self.g.temp(4 * h * w), h, w, 4)
        b = self.g.param(np.zeros(c, np.float32) if bias is None else np.asarray(bias, np.float32))
        self.g.kernel(kname("reef_nchw_to_nhwc4", c=c, hw=h * w), [out.idx, data_idx, b])
        return out

    def stem_conv(self, data_idx: int, c: int, h: int, w: int, co: int, k, stride, pad, *, input_bias=None, **kw) -> Tensor:
        """First convolution of a CNN on the planar input `data` (optionally input + per-channel bias first).
        Tensor-core schedules convert the input to 4-channel channels-last and pad the weights' input channels
        with zeros; the exact-fp32 schedules keep the reference's planar convolution (and its fused_add)."""
        kh, kw_ = (k, k) if isinstance(k, int) else k
        sh = stride if isinstance(stride, int) else stride[0]
        ph = pad if isinstance(pad, int) else pad[0]
        wgt = kw.pop("weight", None)
        if wgt is None:
            wgt = self.he_conv(co, kh, kw_, c)
        attrs4 = dict(ci=4, hi=h, wi=w, co=co, kh=kh, kw=kw_, sh=sh, sw=sh, ph=ph, pw=ph, cr=c)
        op = "fused_nn_conv2d" + ("_add" if kw.get("bias") is not None else "") + ("_nn_relu" if kw.get("relu") else "")
        if self.tc_stem and self.pick_conv_impl(op, attrs4) == 1:
            in_scale = kw.pop("in_scale", None)
            if in_scale is not None:
                wgt = wgt * np.asarray(in_scale, np.float32)[None, None, None, :]
            w4 = np.zeros((co, kh, kw_, 4), np.float32)
            w4[..., :c] = wgt
            x = self.input_nhwc4(data_idx, c, h, w, input_bias)
            return self.conv(x, co, k, stride, pad, weight=w4, real_ci=c, **kw)
        if self.im2col_stem:
            ktot = kh * kw_ * c
            kp = -(-ktot // 32) * 32
            ho, wo = (h + 2 * ph - kh) // sh + 1, (w + 2 * ph - kw_) // sh + 1
            attrs1 = dict(ci=kp, hi=ho, wi=wo, co=co, kh=1, kw=1, sh=1, sw=1, ph=0, pw=0, cr=ktot)
            col = dict(c=c, hi=h, wi=w, kh=kh, kw=kw_, sh=sh, sw=sh, ph=ph, pw=ph, kp=kp)
            if self.pick_conv_impl(op, attrs1) == 1 and self.has_kernel(kname("reef_im2col_nchw", **col)):
                in_scale = kw.pop("in_scale", None)
                if in_scale is not None:
                    wgt = wgt * np.asarray(in_scale, np.float32)[None, None, None, :]
                wcol = np.zeros((co, 1, 1, kp), np.float32)
                wcol[:, 0, 0, :ktot] = wgt.reshape(co, ktot)      # OHWI flattened: k = (ky * kw + kx) * c + channel
                x = Tensor(self.g.temp(ho * wo * kp), ho, wo, kp)
                b = self.g.param(np.zeros(c, np.float32) if input_bias is None else np.asarray(input_bias, np.float32))
                self.g.kernel(kname("reef_im2col_nchw", **col), [x.idx, data_idx, b])
                return self.conv(x, co, 1, 1, 0, weight=wcol, real_ci=ktot, **kw)
        if input_bias is not None:
            x = self.input_bias_nchw(data_idx, c, h, w, input_bias)
        else:
            x = Tensor(data_idx, h, w, c)
        return self.conv(x, co, k, stride, pad, weight=wgt, nchw_in=True, **kw)

    def conv(self, x: Tensor, co: int, k, stride=1, pad=0, *, weight=None,
             out_scale=None, in_scale=None, bias=None, relu=False,
             residual: Tensor | None = None, gamma_beta=None,
             out: Tensor | None = None, nchw_in=False, w_gain: float = 1.0, preact_bias=None, real_ci=None):
        """One convolution kernel.  With ``preact_bias`` (residual convolutions only) the next unit's
        pre-activation relu(out + preact_bias) is produced as well and (out, act) is returned: by the same
        launch where the tensor-core variant exists (reef_conv2d_add_preact), else by a fused_add_nn_relu
        kernel behind the convolution, as in the reference's graphs."""
        kh, kw = (k, k) if isinstance(k, int) else k
        sh, sw = (stride, stride) if isinstance(stride, int) else stride
        ph, pw = (pad, pad) if isinstance(pad, int) else pad
        ci = x.c
        ho = (x.h + 2 * ph - kh) // sh + 1
        wo = (x.w + 2 * pw - kw) // sw + 1
        wgt = self.he_conv(co, kh, kw, ci) if weight is None else weight
        if w_gain != 1.0:
            wgt = wgt * np.float32(w_gain)
        if out_scale is not None:
            wgt = wgt * np.asarray(out_scale, np.float32)[:, None, None, None]
        if in_scale is not None:
            wgt = wgt * np.asarray(in_scale, np.float32)[None, None, None, :]
        if out is None:
            out = self.new_act(ho, wo, co)
        assert (out.h, out.w, out.c) == (ho, wo, co)
        op = "fused_nn_conv2d"
        args = [x.idx, None, out.idx]   # weight slot filled once the variant (and its rounding) is known
        if residual is not None:
            assert (residual.h, residual.w, residual.c) == (ho, wo, co) and residual.cstride == co
            op += "_add"
            args.append(residual.idx)
        if gamma_beta is not None:
            assert bias is None and relu
            op += "_multiply_add"
            args += [self.g.param(gamma_beta[0]), self.g.param(gamma_beta[1])]
        elif bias is not None:
            assert relu, "bias without ReLU is not a family the reference graphs contain"
            op += "_add"
            args.append(self.g.param(bias))
        if relu:
            op += "_nn_relu"
        attrs = dict(ci=ci, hi=x.h, wi=x.w, co=co, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw)
        if nchw_in:
            attrs["nchw"] = 1
        if real_ci is not None and real_ci != ci:
            attrs["cr"] = real_ci      # channels that carry data (the rest is zero padding): roofline bookkeeping
        if x.cstride != ci or x.coff:
            attrs["ics"] = x.cstride
            attrs["ioff"] = x.coff
        if out.cstride != co or out.coff:
            attrs["ocs"] = out.cstride
            attrs["ooff"] = out.coff
        if preact_bias is not None:
            assert op == "fused_nn_conv2d_add" and out.cstride == co and not out.coff
            if self.pick_conv_impl("reef_conv2d_add_preact", attrs) == 1:
                act = self.new_act(ho, wo, co)
                args[1] = self.g.param(round_tf32(wgt))
                args += [self.g.param(preact_bias), act.idx]
                full = kname("reef_conv2d_add_preact", **attrs, v=1)
                self.g.kernel(kname("reef_conv2d_add_preact", **attrs, v=1, **tuned_plan(full)), args)
                return out, act
        impl = self.pick_conv_impl(op, attrs)
        if impl:
            attrs["v"] = impl
            # the tensor core reads 19 bits of each fp32 operand; weights of tensor-core layers are stored
            # already rounded to the nearest TF32 value, so the model in the .param file is exactly the
            # model the hardware multiplies with (and the oracle reads the same bytes)
            wgt = round_tf32(wgt)
            attrs.update(tuned_plan(kname(op, **attrs)))
        args[1] = self.g.param(wgt)
        self.g.kernel(kname(op, **attrs), args)
        if preact_bias is not None:
            return out, self.bias_relu(out, preact_bias)
        return out

    @staticmethod
    def has_kernel(name: str) -> bool:
        from .. import capi
        try:
            capi.kernel_plan(name)
            return True
        except capi.ReefError:
            return False

    def pick_conv_impl(self, op, attrs) -> int:
        """0 = fp32 implicit GEMM on CUDA cores; 1 = tcgen05 TF32 implicit GEMM (fp32 accumulate).
        ``conv_impl``: "simt" forces 0, "auto"/"tc" asks the kernel registry whether variant 1
        supports the shape (channels a multiple of 32, stride 1 or 2, channels-last input) and
        falls back to 0 otherwise."""
        if self.conv_impl == "simt":
            return 0
        from .. import capi
        try:
            capi.kernel_plan(kname(op, **attrs, v=1))
            return 1
        except capi.ReefError:
            return 0

    def pool(self, x: Tensor, kind: str, k: int, stride: int, pad: int, *,
             bias=None, out: Tensor | None = None, count_include_pad=True, ceil_mode=False) -> Tensor:
        if ceil_mode:
            ho = -(-(x.h + 2 * pad - k) // stride) + 1
            wo = -(-(x.w + 2 * pad - k) // stride) + 1
        else:
            ho = (x.h + 2 * pad - k) // stride + 1
            wo = (x.w + 2 * pad - k) // stride + 1
        if out is None:
            out = self.new_act(ho, wo, x.c)
        attrs = dict(c=x.c, hi=x.h, wi=x.w, k=k, s=stride, p=pad, ho=ho, wo=wo)
        if x.cstride != x.c or x.coff:
            attrs["ics"] = x.cstride
            attrs["ioff"] = x.coff
        if out.cstride != x.c or out.coff:
            attrs["ocs"] = out.cstride
            attrs["ooff"] = out.coff
        if kind == "max":
            op = "fused_nn_max_pool2d"
            args = [x.idx, out.idx]
            if bias is not None:
                op += "_add_nn_relu"
                args.append(self.g.param(bias))
        else:
            op = "fused_nn_avg_pool2d"
            attrs["cip"] = 1 if count_include_pad else 0
            args = [x.idx, out.idx]
        self.g.kernel(kname(op, **attrs), args)
        return out

    def bias_relu(self, x: Tensor, bias) -> Tensor:
        assert x.cstride == x.c and x.coff == 0
        out = self.new_act(x.h, x.w, x.c)
        self.g.kernel(kname("fused_add_nn_relu", c=x.c, n=x.h * x.w),
                      [out.idx, x.idx, self.g.param(bias)])
        return out

    def bias_relu_slice(self, x: Tensor, bias) -> Tensor:
        """relu(x + bias) on a channel slice view (DenseNet pre-activation)."""
        out = self.new_act(x.h, x.w, x.c)
        attrs = dict(c=x.c, n=x.h * x.w)
        if x.cstride != x.c or x.coff:
            attrs["ics"] = x.cstride
            attrs["ioff"] = x.coff
        self.g.kernel(kname("fused_add_nn_relu", **attrs), [out.idx, x.idx, self.g.param(bias)])
        return out

    def global_avg_pool(self, x: Tensor) -> Tensor:
        assert x.cstride == x.c and x.coff == 0
        out = Tensor(self.g.temp(x.c), 1, 1, x.c)
        self.g.kernel(kname("fused_nn_global_avg_pool2d", c=x.c, hw=x.h * x.w), [x.idx, out.idx])
        return out

    def flatten(self, x: Tensor) -> Tensor:
        n = x.h * x.w * x.c
        out = Tensor(self.g.temp(n), 1, 1, n)
        self.g.kernel(kname("fused_nn_batch_flatten", n=n), [out.idx, x.idx])
        return out

    def dense(self, x: Tensor, n: int, *, relu=False, w_std=None, weight=None, bias=None,
              out_idx=None) -> Tensor:
        k = x.h * x.w * x.c
        if weight is None:
            std = np.sqrt(2.0 / k) if w_std is None else w_std
            weight = self.rng().normal(0.0, std, (n, k)).astype(np.float32)
        if bias is None:
            bias = self.rng().normal(0.0, 0.1, n).astype(np.float32)
        out = Tensor(self.g.temp(n) if out_idx is None else out_idx, 1, 1, n)
        op = "fused_nn_dense_add" + ("_nn_relu" if relu else "")
        self.g.kernel(kname(op, k=k, n=n), [x.idx, self.g.param(weight), out.idx, self.g.param(bias)])
        return out

    def softmax_output(self, x: Tensor) -> int:
        n = x.h * x.w * x.c
        out = self.g.add_storage("output", n)   # not in "args": the reference lists inputs and params only
        self.g.kernel(kname("fused_nn_softmax", n=n), [x.idx, out])
        return out
