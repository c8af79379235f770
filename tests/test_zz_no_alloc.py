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
    outs = dict(
        dx=torch.empty_like(x), dw_in=torch.empty_like(w_in), db_in=torch.empty_like(b_in),
        dw_hid=torch.empty_like(w_hid), db_hid=torch.empty_like(b_hid), dw_out=torch.empty_like(w_out),
        db_out=torch.empty_like(b_out),
    )  # fmt: skip
    head = (x.data_ptr(), d_in, w_in.data_ptr(), b_in.data_ptr(), w_hid.data_ptr(), b_hid.data_ptr(),
            w_out.data_ptr(), b_out.data_ptr(), go.data_ptr(), d_out, outs["dx"].data_ptr(), d_in,
            outs["dw_in"].data_ptr(), outs["db_in"].data_ptr(), outs["dw_hid"].data_ptr(), outs["db_hid"].data_ptr(),
            outs["dw_out"].data_ptr(), outs["db_out"].data_ptr())  # fmt: skip
    tail = (rows, d_in, d_hid, d_out, depth, _lib.ACTIVATION_CODE["relu"], _lib.DTYPE_CODE[x.dtype], 0,
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    lib = _lib.lib()
    if entry == "static":
        _lib.check(lib.th_mlp_bwd_static(*head, *tail), "th_mlp_bwd_static")
    else:
        _lib.check(lib.th_mlp_bwd(*head, workspace.data_ptr(), workspace.numel(), *tail), "th_mlp_bwd")
    torch.cuda.synchronize()
    return outs


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


def test_static_scratch_backward_refuses_networks_beyond_its_buffer():
    lib = _lib.lib()
    depth = 20  # 19 hidden 64 x 64 layers: 77 824 + ... floats > 65 536
    assert lib.th_mlp_workspace_bytes(64, 64, 64, depth) > lib.th_mlp_bwd_static_max_bytes()
    z = torch.zeros(64, dtype=torch.float16, device="cuda")
    args = [z.data_ptr()] * 18
    args[1], args[9], args[11] = 64, 64, 64
    rc = lib.th_mlp_bwd_static(*args, 0, 64, 64, 64, depth, 1, 1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"built-in buffer" in lib.th_last_error_string()
