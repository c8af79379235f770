r"""The scratch-free MLP backward (``th_mlp_bwd_static``) against the regular entry point.

Collected last on purpose (the ``zz`` in the file name): a run that stops at the first failure
has then already been through every other test.

``th_mlp_bwd_static`` is for callers that cannot provide device scratch at call time — a plug-in
whose host application owns all device memory, a loop that must not trigger an allocation's
device-wide synchronisation, a C caller without an allocator.  It keeps its fp32 partial sums in
a 256 KB array inside the library image instead.  That array is shared by all calls and still
holds the previous call's sums, so the test calls it twice in a row with different gradients and
checks both results against ``th_mlp_bwd`` given freshly allocated scratch.  Both entry points
are called directly through the C ABI.
"""
import pytest
import torch

from triton_helpers_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = 2e-3  # the tight float16 tolerance of the fused-MLP tests (fp32 partial sums, atomics reorder them)


def nerr(got, want) -> float:
    got, want = got.double(), want.double()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-300))


def run_backward(entry, x, go, params, shape, workspace=None):
    d_in, d_hid, d_out, depth = shape
    w_in, b_in, w_hid, b_hid, w_out, b_out = params
    rows = x.shape[0]
    like = lambda t: None if t is None else torch.empty_like(t)  # noqa: E731
    outs = dict(dx=like(x), dw_in=like(w_in), db_in=like(b_in), dw_hid=like(w_hid), db_hid=like(b_hid), dw_out=like(w_out),
                db_out=like(b_out))  # fmt: skip
    ptr = _lib.ptr
    head = (x.data_ptr(), d_in, w_in.data_ptr(), ptr(b_in), ptr(w_hid), ptr(b_hid), w_out.data_ptr(), ptr(b_out), go.data_ptr(),
            d_out, outs["dx"].data_ptr(), d_in, outs["dw_in"].data_ptr(), ptr(outs["db_in"]), ptr(outs["dw_hid"]),
            ptr(outs["db_hid"]), outs["dw_out"].data_ptr(), ptr(outs["db_out"]))  # fmt: skip
    tail = (rows, d_in, d_hid, d_out, depth, _lib.ACTIVATION_CODE["relu"], _lib.DTYPE_CODE[x.dtype], 0,
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    lib = _lib.lib()
    if entry == "static":
        _lib.check(lib.th_mlp_bwd_static(*head, *tail), "th_mlp_bwd_static")
    else:
        _lib.check(lib.th_mlp_bwd(*head, workspace.data_ptr(), workspace.numel(), *tail), "th_mlp_bwd")
    torch.cuda.synchronize()
    return {k: v for k, v in outs.items() if v is not None}


def test_static_scratch_backward_matches_regular_backward_twice():
    shape = (32, 64, 16, 4)
    d_in, d_hid, d_out, depth = shape
    dtype = torch.float16
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device="cuda", generator=g) * scale).to(dtype)  # noqa: E731
    params = (rnd(d_hid, d_in, scale=d_in**-0.5), rnd(d_hid, scale=0.1), rnd((depth - 1) * d_hid, d_hid, scale=d_hid**-0.5),
              rnd(depth - 1, d_hid, scale=0.1), rnd(d_out, d_hid, scale=d_hid**-0.5), rnd(d_out, scale=0.1))  # fmt: skip
    rows = 5000
    x = rnd(rows, d_in)
    ws_bytes = _lib.lib().th_mlp_workspace_bytes(*shape)
    assert 0 < ws_bytes <= _lib.lib().th_mlp_bwd_static_max_bytes() == 256 * 1024
    for call in range(2):  # the second call finds the first call's sums in the shared scratch
        go = rnd(rows, d_out, scale=0.1 * (call + 1))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        want = run_backward("regular", x, go, params, shape, workspace)
        got = run_backward("static", x, go, params, shape)
        assert torch.equal(got["dx"], want["dx"]), f"call {call}: dx does not depend on the scratch at all"
        for name in want:
            assert nerr(got[name].float(), want[name].float()) <= TOL, f"call {call}: {name} {nerr(got[name].float(), want[name].float())}"


def test_static_scratch_on_the_tensor_core_path_and_after_a_larger_network():
    # A bias-free ReLU network takes the tcgen05 backward, whose CTAs flush their tensor-memory weight gradients
    # into the scratch with float32 reductions - the path that depends most on the scratch starting at zero.
    # Called right after the LARGER biased network of the test above has left its sums in the shared array, twice,
    # with a row count that ends inside a 128-row tile; checked against th_mlp_bwd AND against the CPU oracle.
    from oracle import fused_mlp as oracle

    dtype = torch.float16
    g = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device="cuda", generator=g) * scale).to(dtype)  # noqa: E731
    big = (32, 64, 16, 4)
    big_params = (rnd(64, 32, scale=32**-0.5), rnd(64, scale=0.1), rnd(192, 64, scale=0.125), rnd(3, 64, scale=0.1),
                  rnd(16, 64, scale=0.125), rnd(16, scale=0.1))  # fmt: skip
    run_backward("static", rnd(1000, 32), rnd(1000, 16), big_params, big)  # leaves 15 632 non-zero sums behind
    shape = (32, 64, 16, 2)
    d_in, d_hid, d_out, depth = shape
    params = (rnd(d_hid, d_in, scale=d_in**-0.5), None, rnd(d_hid, d_hid, scale=d_hid**-0.5), None,
              rnd(d_out, d_hid, scale=d_hid**-0.5), None)  # fmt: skip
    rows = 128 * 9 + 45
    x = rnd(rows, d_in)
    ws_bytes = _lib.lib().th_mlp_workspace_bytes(*shape)
    for call in range(2):
        go = rnd(rows, d_out, scale=0.1 * (call + 1))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        want = run_backward("regular", x, go, params, shape, workspace)
        got = run_backward("static", x, go, params, shape)
        ref = oracle.forward_backward_storage_rounded(x.cpu().unsqueeze(0), params[0].cpu(), None, params[4].cpu(), None,
                                                      params[2].cpu(), None, go.float().cpu().unsqueeze(0))  # fmt: skip
        assert torch.equal(got["dx"], want["dx"])
        for name, oracle_grad in (("dw_in", ref[2]), ("dw_out", ref[4]), ("dw_hid", ref[6])):
            assert nerr(got[name].float(), want[name].float()) <= TOL, f"call {call}: {name} against th_mlp_bwd"
            assert nerr(got[name].float().cpu(), oracle_grad) <= 1e-2, f"call {call}: {name} against the oracle"
    assert _lib.lib().th_mlp_tc_status() == 0


def test_static_scratch_backward_refuses_networks_beyond_its_buffer():
    lib = _lib.lib()
    depth = 20  # 19 hidden 64 x 64 layers: 77 824 + ... floats > 65 536
    assert lib.th_mlp_workspace_bytes(64, 64, 64, depth) > lib.th_mlp_bwd_static_max_bytes()
    z = torch.zeros(64, dtype=torch.float16, device="cuda")
    args = [z.data_ptr()] * 18
    args[1], args[9], args[11] = 64, 64, 64
    rc = lib.th_mlp_bwd_static(*args, 0, 64, 64, 64, depth, 1, 1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"built-in buffer" in lib.th_last_error_string()
