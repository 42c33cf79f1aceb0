"""A cross-GPU wait that runs out, on one GPU and without any fault: the peer's flag is simply never written.  The
kernel must return within its budget, leave its status code in the status word (which ``check_status`` turns into an
exception) and must not have touched the state that depended on the missing peer."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_RANKS = 8


@pytest.fixture
def native():
    from b200moe.ops import native as nat
    nat.require()
    nat.clear_status()
    nat.set_wait_seconds(0.002)
    yield nat
    nat.clear_status()
    nat.set_wait_seconds(10.0)


def _table(*tensors):
    ptrs = [t.data_ptr() for t in tensors] + [0] * (MAX_RANKS - len(tensors))
    return (ctypes.c_ulonglong * MAX_RANKS)(*ptrs)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_combine_kernel_gives_up_and_reports_its_code(native):
    """The source side of the expert exchange waiting for an owner that never delivers."""
    pad = torch.zeros(32 * MAX_RANKS, dtype=torch.int32, device="cuda")       # nobody ever signals
    status = native.status_word()
    tokens, D = 64, 128
    ret = torch.ones(2 * tokens, D, dtype=torch.bfloat16, device="cuda")
    out = torch.full((tokens, D), 7.0, dtype=torch.bfloat16, device="cuda")
    t0 = time.perf_counter()
    native._call("b2_ep_combine", ctypes.c_void_p(ret.data_ptr()), ctypes.c_void_p(0), ctypes.c_void_p(out.data_ptr()),
                 ctypes.c_void_p(0), ctypes.c_int(tokens), ctypes.c_int(D), ctypes.c_void_p(pad.data_ptr()),
                 ctypes.c_int(18), ctypes.c_int(2), ctypes.c_int(1), ctypes.c_void_p(status.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 104
    assert float(out.float().min()) == 7.0              # the output was left alone
    with pytest.raises(RuntimeError, match="104"):
        native.check_status()
    native.clear_status()
    assert native.check_status() == 0


def test_end_of_step_kernel_leaves_master_and_moments_alone_when_a_rank_never_arrives(native):
    n = 4096
    full_g = torch.randn(2 * n, device="cuda")
    full_w = torch.zeros(2 * n, dtype=torch.bfloat16, device="cuda")
    pad = torch.zeros(32 * MAX_RANKS, dtype=torch.int32, device="cuda")
    entries = torch.tensor([[0, 0, n, 0]], dtype=torch.int64, device="cuda")
    master, m, v = torch.randn(n, device="cuda"), torch.rand(n, device="cuda"), torch.rand(n, device="cuda")
    shard_grad = torch.zeros(n, device="cuda")
    before = [t.clone() for t in (master, m, v, shard_grad, full_w)]
    counter = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = native.status_word()
    # rank 0 of an emulated pair whose other member never launches: its flag [slot][1] stays 0
    native._call("b2_fsdp_step", _table(full_g, full_g), _table(full_w, full_w), _table(pad, pad),
                 ctypes.c_void_p(entries.data_ptr()), ctypes.c_int(1), ctypes.c_int(0), ctypes.c_int(2),
                 ctypes.c_int(1), ctypes.c_int(8), ctypes.c_void_p(master.data_ptr()), ctypes.c_void_p(m.data_ptr()),
                 ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(shard_grad.data_ptr()), ctypes.c_float(1e-3),
                 ctypes.c_float(0.9), ctypes.c_float(0.999), ctypes.c_float(1e-8), ctypes.c_float(0.01),
                 ctypes.c_float(1e-3), ctypes.c_int(1), ctypes.c_int(0), ctypes.c_void_p(counter.data_ptr()),
                 ctypes.c_void_p(status.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 105
    for now, then in zip((master, m, v, shard_grad, full_w), before):
        assert torch.equal(now, then)
    assert int(counter[0].item()) == 0          # the block counter is back at zero for the next launch
    # the "leave" flag was not raised: the other rank must not take this one for finished
    assert int(pad.view(32, MAX_RANKS)[9, 0].item()) == 0
    native.clear_status()


def test_vectorised_end_of_step_kernel_matches_the_adamw_rule_on_emulated_single_rank(native):
    native.set_wait_seconds(5.0)
    n = 8 * 1000
    full_g = torch.randn(n, device="cuda")
    full_w = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    pad = torch.zeros(32 * MAX_RANKS, dtype=torch.int32, device="cuda")
    entries = torch.tensor([[0, 0, n - 64, 0], [n - 64, n - 64, 64, 0]], dtype=torch.int64, device="cuda")
    master, m, v = torch.randn(n, device="cuda"), torch.rand(n, device="cuda") * 0.1, torch.rand(n, device="cuda")
    shard_grad = torch.zeros(n, device="cuda")
    p0, m0, v0 = master.clone(), m.clone(), v.clone()
    counter = torch.zeros(8, dtype=torch.int32, device="cuda")
    lr, b1, b2, eps, wd, a_t = 1e-2, 0.9, 0.999, 1e-8, 0.01, 3e-3
    native._call("b2_fsdp_step", _table(full_g), _table(full_w), _table(pad), ctypes.c_void_p(entries.data_ptr()),
                 ctypes.c_int(2), ctypes.c_int(0), ctypes.c_int(1), ctypes.c_int(1), ctypes.c_int(8),
                 ctypes.c_void_p(master.data_ptr()), ctypes.c_void_p(m.data_ptr()), ctypes.c_void_p(v.data_ptr()),
                 ctypes.c_void_p(shard_grad.data_ptr()), ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2),
                 ctypes.c_float(eps), ctypes.c_float(wd), ctypes.c_float(a_t), ctypes.c_int(1), ctypes.c_int(0),
                 ctypes.c_void_p(counter.data_ptr()), ctypes.c_void_p(native.status_word().data_ptr()), _stream())
    torch.cuda.synchronize()
    assert native.check_status() == 0
    g = full_g
    want_m = b1 * m0 + (1 - b1) * g
    want_v = b2 * v0 + (1 - b2) * g * g
    want_p = p0 * (1 - lr * wd) - a_t * want_m / (want_v.sqrt() + eps)
    torch.testing.assert_close(shard_grad, g)
    torch.testing.assert_close(m, want_m, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(v, want_v, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(master, want_p, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(full_w.float(), want_p.bfloat16().float())


def _pp_send(native, src, dst, flag, ack, seq, need_ack, wait_s, ticket, status):
    native._call("b2_pp_send", ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()),
                 ctypes.c_longlong(src.numel() * src.element_size()), ctypes.c_void_p(flag.data_ptr()),
                 ctypes.c_void_p(ack.data_ptr()), ctypes.c_int(seq), ctypes.c_int(need_ack),
                 ctypes.c_longlong(int(wait_s * 1e9)), ctypes.c_void_p(ticket.data_ptr()),
                 ctypes.c_void_p(status.data_ptr()), _stream())


def test_pipeline_link_kernels_deliver_and_give_up(native):
    """The pipeline's send / wait / acknowledge kernels with this GPU as its own neighbour: a message lands whole and
    its number is published; a send into a full ring and a wait for a message that nobody sends both return within
    their budget with their status code, and the send leaves slot and flag alone."""
    status = native.status_word()
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    words = torch.zeros(64, dtype=torch.int32, device="cuda")
    for numel in (8, 4096 * 33 + 8, 64 * 1024 * 1024 + 24):            # bf16 elements: whole 16-byte units
        src = torch.randn(numel, device="cuda").bfloat16()
        dst = torch.zeros(numel + 64, dtype=torch.bfloat16, device="cuda")
        words.zero_()
        _pp_send(native, src, dst, words[3:], words[32:], 5, 0, 0.2, ticket, status)
        native._call("b2_pp_wait", ctypes.c_void_p(words[3:].data_ptr()), ctypes.c_int(5),
                     ctypes.c_longlong(200_000_000), ctypes.c_void_p(status.data_ptr()), _stream())
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(dst[:numel], src) and float(dst[numel:].float().abs().max()) == 0.0
        assert int(words[3].item()) == 5 and int(ticket.item()) == 0
    # acknowledge: both neighbours' words
    native._call("b2_pp_ack", ctypes.c_void_p(words[32:].data_ptr()), ctypes.c_void_p(words[33:].data_ptr()),
                 ctypes.c_int(9), _stream())
    native._call("b2_pp_ack", ctypes.c_void_p(0), ctypes.c_void_p(words[40:].data_ptr()), ctypes.c_int(4), _stream())
    torch.cuda.synchronize()
    assert words[32:34].tolist() == [9, 9] and int(words[40].item()) == 4
    # a send that has room once message 9 is acknowledged goes through; one that needs message 10 gives up
    src = torch.randn(4096, device="cuda").bfloat16()
    dst = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    _pp_send(native, src, dst, words[4:], words[32:], 11, 9, 0.2, ticket, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(dst, src) and int(words[4].item()) == 11
    dst.zero_()
    t0 = time.perf_counter()
    _pp_send(native, src, dst, words[5:], words[32:], 12, 10, 0.05, ticket, status)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 321
    assert float(dst.float().abs().max()) == 0.0 and int(words[5].item()) == 0 and int(ticket.item()) == 0
    native.clear_status()
    t0 = time.perf_counter()
    native._call("b2_pp_wait", ctypes.c_void_p(words[6:].data_ptr()), ctypes.c_int(1), ctypes.c_longlong(50_000_000),
                 ctypes.c_void_p(status.data_ptr()), _stream())
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 322
    with pytest.raises(RuntimeError, match="322"):
        native.check_status()
    native.clear_status()
    # misuse is refused on the host
    with pytest.raises(RuntimeError, match="-8"):
        _pp_send(native, src[:4], dst, words[5:], words[32:], 13, 0, 0.05, ticket, status)
