"""Convolution test cases shared by the CPU pins and the GPU parity tests (no torch, no GPU): geometry from the golden
file, a vectorised im2col index map, and the inputs of the reference's own int8 convolution tests."""
import numpy as np


def conv_geometry_from_golden(row):
    """ConvGeometry + group index from a ``conv_<i>_geom`` row of the golden file (the 21 members of tqt_conv_params
    in declaration order, then the group index)."""
    from oracle.tqo import ConvGeometry
    r = [int(x) for x in row]
    g = ConvGeometry(r[18], r[19], r[20], r[0:3], r[6:9], r[9:12], r[12:15], r[15:18])
    assert list(g.output_shape) == r[3:6]
    return g, r[21]


def im2col_index(geom, channel_first, group_idx=0):
    """[rows, K] flat indices into the activation tensor ([C,D,H,W] or [D,H,W,C]) for every cell of the im2col
    matrix, -1 inside the padding.  Vectorised index arithmetic, independent of the oracle's loops."""
    ID, IH, IW = geom.input_shape
    OD, OH, OW = geom.output_shape
    KD, KH, KW = geom.kernel_shape
    ic_pg = geom.input_channel // geom.groups
    pos = np.arange(geom.rows)
    ow, oh, od = pos % OW, (pos // OW) % OH, pos // (OW * OH)
    k = np.arange(geom.k)
    kvol = KD * KH * KW
    if channel_first:
        ic, kpos = k // kvol, k % kvol
    else:
        kpos, ic = k // ic_pg, k % ic_pg
    kw, kh, kd = kpos % KW, (kpos // KW) % KH, kpos // (KW * KH)
    i_d = od[:, None] * geom.stride[0] + kd[None, :] * geom.dilation[0] - geom.pad[0]
    i_h = oh[:, None] * geom.stride[1] + kh[None, :] * geom.dilation[1] - geom.pad[1]
    i_w = ow[:, None] * geom.stride[2] + kw[None, :] * geom.dilation[2] - geom.pad[2]
    ok = (i_d >= 0) & (i_d < ID) & (i_h >= 0) & (i_h < IH) & (i_w >= 0) & (i_w < IW)
    sp = (i_d * IH + i_h) * IW + i_w
    c = group_idx * ic_pg + ic[None, :]
    idx = c * (ID * IH * IW) + sp if channel_first else sp * geom.input_channel + c
    return np.where(ok, idx, -1)


def conv_acceptance_case(oracle, geom, channel_first, group_idx=0):
    """Inputs of the reference's own tests of the int8 convolution wrappers (test/common/quantized_conv_test_runner.h:
    channel-first :147-262, channel-last packed :509-618): activation and weights ~ U(-1,1) from one mt19937(42)
    stream, bias ~ U(-10,10) seed 123; the activation quantised asymmetrically per tensor, the weights symmetrically
    per output channel, the bias to int32 with the activation zero point fused in; output scale / zero point from the
    range of the real-valued convolution.  ``real``: [positions, channels] (channel-last) or [channels, positions]."""
    f32 = np.float32
    n_act = int(np.prod(geom.input_shape)) * geom.input_channel
    oc = geom.output_channel // geom.groups
    K = geom.k
    stream = oracle.fill_uniform((n_act + oc * K,), np.float32, -1.0, 1.0, 42)
    act, W = stream[:n_act], stream[n_act:].reshape(oc, K)
    bias = oracle.fill_uniform((oc,), np.float32, -10.0, 10.0, 123)
    idx = im2col_index(geom, channel_first, group_idx)
    col = np.where(idx >= 0, act[np.maximum(idx, 0)], f32(0)).astype(np.float64)     # [rows, K]
    real = col @ W.T.astype(np.float64) + bias.astype(np.float64)[None, :]           # [rows, oc]
    real = (real.T if channel_first else real).astype(f32)

    def asym(x):
        fmin, fmax = f32(min(x.min(), 0.0)), f32(max(x.max(), 0.0))
        sc = f32(f32(fmax - fmin) / f32(255.0))
        if sc == 0:
            return f32(1.0), 0
        zp = int(np.rint(f32(-128.0) - f32(fmin / sc)))
        return sc, (-127 if zp == -128 else zp)

    def quant(x, sc, zp):
        return np.clip(np.rint((x / f32(sc)).astype(f32)) + f32(zp), -128, 127).astype(np.int8)

    s_act, zp_act = asym(act)
    absmax = np.abs(W).max(axis=1).astype(f32)
    s_w = (f32(2.0) * absmax / f32(255.0)).astype(f32)
    s_w[s_w == 0] = 1.0
    act_q = quant(act, s_act, zp_act)
    W_q = np.stack([quant(W[j], s_w[j], 0) for j in range(oc)])
    bias_i32 = np.clip(np.rint((bias / (f32(s_act) * s_w)).astype(f32)), -2147483648.0, 2147483647.0).astype(np.int64).astype(np.int32)
    fused = oracle.fuse_zp_to_bias(bias_i32, W_q, zp_act)
    sd, zpd = asym(real)
    return dict(act=act_q, W=W_q, scale_act=float(s_act), zp_act=zp_act, scale_w=s_w, bias_fused=fused, scale_d=float(sd),
                zp_d=zpd, real=real)
