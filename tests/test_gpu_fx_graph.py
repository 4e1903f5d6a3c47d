"""Hand-built FX ``GraphModule``s with the node patterns the reference's ``convert_pt2e`` emits,
executed on the GPU through the registered operators, eagerly and from a CUDA graph.

(i) a microscaling site (reference ``quantization/quantize_pt2e.py:869-923, 1035-1057``): the
activation goes through ``quantize_mx(x, <get_attr qmap>, ch_axis, bs, qmax, pot, scale_qmap,
quant_code)`` and two ``getitem``s; the weight is baked into ``<w>_<dtype>`` / ``<w>_scale``
buffers; the consumer is ``linear_mx`` with keyword arguments in the converter's order.
(ii) a per-tensor FP8 site (``:526-626``): ``quantize(x, <get_attr scale>, None, None, None,
<get_attr qmap>)`` -> ``aten.linear`` on the baked weight codes -> ``dequantize(y, <get_attr
s_a * s_w>, None, None, None, <get_attr out-dtype qmap>)``.
"""

import operator

import pytest
import torch
from torch import fx

import cases as C
from golden_io import bits_equal, describe_mismatch, golden_cases
from oracle import quantizers as OQ
from oracle import tables as OT

pytestmark = pytest.mark.gpu
Q = torch.ops.quantized_ops


def _vb():
    import voyager_b200

    return voyager_b200


def rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def _module_with(buffers):
    root = torch.nn.Module()
    for name, value in buffers.items():
        root.register_buffer(name, value)
    return root


def mx_linear_graph(vb, weight, qmap, block_size, quant_max, pot):
    """``x -> quantize_mx -> getitem 0/1 -> linear_mx`` against a weight quantized once into buffers."""
    w_scale, w_codes = Q.quantize_mx(weight, qmap, [-1], block_size, quant_max, pot)
    root = _module_with({"qmap": qmap, "weight_int8": w_codes, "weight_scale": w_scale})
    g = fx.Graph()
    x = g.placeholder("x")
    qmap_node = g.get_attr("qmap")
    qmx = g.call_function(Q.quantize_mx.default, (x, qmap_node, (-1,), block_size, quant_max, pot, None, None))
    qmx.meta["dtype"] = ("fp8_e8m0", "int8")
    scale = g.call_function(operator.getitem, (qmx, 0))
    codes = g.call_function(operator.getitem, (qmx, 1))
    w = g.get_attr("weight_int8")
    w.meta["dtype"] = "int8"
    ws = g.get_attr("weight_scale")
    y = g.call_function(Q.linear_mx.default, (codes, w, None),
                        {"input_scale": scale, "weight_scale": ws, "block_size": block_size})
    g.output((scale, codes, y))
    return fx.GraphModule(root, g)


def fp8_linear_graph(vb, weight, s_act, s_w):
    """``x -> quantize -> aten.linear -> dequantize`` with the weight cast in place at convert time."""
    e4m3 = vb.get_quantization_map("fp8_e4m3", "cuda")
    ident = vb.get_quantization_map(None, "cuda")
    w_codes = Q.quantize(weight, s_w, None, None, None, e4m3)
    root = _module_with({"qmap": e4m3, "qmap_1": ident, "weight": w_codes, "linear_scale": s_act,
                         "linear_scale_1": s_act * s_w})
    g = fx.Graph()
    x = g.placeholder("x")
    q = g.call_function(Q.quantize.default, (x, g.get_attr("linear_scale"), None, None, None, g.get_attr("qmap")))
    q.meta["dtype"] = "fp8_e4m3"
    y = g.call_function(torch.ops.aten.linear.default, (q, g.get_attr("weight")))
    dq = g.call_function(Q.dequantize.default, (y, g.get_attr("linear_scale_1"), None, None, None, g.get_attr("qmap_1")))
    g.output((q, dq))
    return fx.GraphModule(root, g)


def _replay_from_cuda_graph(module, x):
    """Outputs of ``module(x)`` captured into a CUDA graph and replayed on fresh input bytes."""
    static_x = torch.zeros_like(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        module(static_x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = module(static_x)
    static_x.copy_(x)
    graph.replay()
    torch.cuda.synchronize()
    return out


def test_mx_site_runs_as_an_fx_graph_and_from_a_cuda_graph():
    vb = _vb()
    op, args, kwargs, expected = golden_cases(OT.quantization_map)["linear_mx_int8"]
    x, w, _ = args
    gm = mx_linear_graph(vb, w.cuda(), vb.get_quantization_map("int8", "cuda"), 16, 127.0, True)
    gm.graph.lint()
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert targets == [Q.quantize_mx.default, operator.getitem, operator.getitem, Q.linear_mx.default]
    for got in (gm(x.cuda()), _replay_from_cuda_graph(gm, x.cuda())):
        scale, codes, y = (t.cpu() for t in got)
        vb.ops.gemm_status()
        assert bits_equal(scale, expected[0]), describe_mismatch(scale, expected[0])
        assert bits_equal(codes, expected[1]), describe_mismatch(codes, expected[1])
        assert y.shape == expected[4].shape and y.dtype == expected[4].dtype
        assert rel_err(y, expected[4]) <= 1e-2, rel_err(y, expected[4])
    # the baked weight buffers are the golden weight codes and scales
    assert bits_equal(gm.weight_scale.cpu(), expected[2]) and bits_equal(gm.weight_int8.cpu(), expected[3])


def test_per_tensor_fp8_site_runs_as_an_fx_graph_and_from_a_cuda_graph():
    vb = _vb()
    x = C.randn(301, 64, 256, std=1.5, outliers=0.001)
    w = C.randn(302, 96, 256, std=0.02)
    s_act = (x.abs().amax() / 448.0)
    s_w = (w.abs().amax() / 448.0)
    e4m3, ident = OT.quantization_map("fp8_e4m3"), OT.quantization_map(None)
    want_q = OQ.quantize(x, s_act, None, None, None, e4m3)
    want = OQ.dequantize(torch.nn.functional.linear(want_q, OQ.quantize(w, s_w, None, None, None, e4m3)),
                         s_act * s_w, None, None, None, ident)
    gm = fp8_linear_graph(vb, w.cuda(), s_act.cuda(), s_w.cuda())
    gm.graph.lint()
    for got in (gm(x.cuda()), _replay_from_cuda_graph(gm, x.cuda())):
        q, y = (t.cpu() for t in got)
        assert bits_equal(q, want_q), describe_mismatch(q, want_q)
        assert y.shape == want.shape and y.dtype == want.dtype
        # one bfloat16 GEMM each side (cuBLAS here, the CPU's in the oracle): accumulation order only
        assert rel_err(y, want) <= 1e-2, rel_err(y, want)


def test_voyager_gpu_operators_match_the_functions_they_wrap():
    """The ``voyager_gpu`` call targets of a lowered graph (reference ``backend/gpu/nvfp4.py:675-1152``,
    ``fp8.py:311-340``) give what the package's own functions give."""
    vb = _vb()
    G = torch.ops.voyager_gpu
    x = C.randn(310, 256, 128, outliers=0.002).cuda()
    w = C.randn(311, 192, 128, std=0.02).cuda()
    codes, scales, t = G.cast_nvfp4(x, None, None, 1)
    c2, s2, t2 = vb.nvfp4.quantize_nvfp4(x)
    assert torch.equal(codes, c2) and torch.equal(scales, s2.reshape(-1)) and torch.equal(t, t2)
    assert scales.dim() == 1 and codes.shape == (256, 64) and t.dim() == 0 and t.dtype == torch.bfloat16
    ct, st, tt = G.cast_nvfp4(x, None, None, 0)
    assert ct.shape == (128, 128)
    pair = G.cast_nvfp4_pair(x, None, None, None)
    assert torch.equal(pair[0], codes) and torch.equal(pair[3], ct) and torch.equal(pair[4], st)
    sq = G.cast_nvfp4_square(w)
    assert sq[0].shape == (192, 64) and sq[2].shape == (128, 96) and sq[4].dim() == 0
    wc, ws, tw = G.cast_nvfp4(w, None, None, 1)
    alpha = (t * tw).float()
    one = torch.ones((), device="cuda")
    y = G.nvfp4_linear(codes, scales, wc, ws, alpha, one, None)
    want = vb.nvfp4.emulate_nvfp4_linear(codes, scales, wc, ws, alpha, one, None)
    vb.ops.gemm_status()
    assert y.shape == (256, 192) and y.dtype == torch.bfloat16
    assert rel_err(y, want) <= 1e-2
    s = (x.abs().amax() / 448.0).to(torch.bfloat16)
    c8, c8t, amax = G.cast_transpose_fp8(x, s, torch.float8_e4m3fn)
    assert c8.dtype == torch.float8_e4m3fn and c8t.shape == (128, 256)
    assert torch.equal(c8.view(torch.uint8), vb.fp8.quantize_fp8(x, s)) and torch.equal(c8t.view(torch.uint8),
                                                                                        c8.view(torch.uint8).t())
    assert float(amax) == float(x.abs().amax())
