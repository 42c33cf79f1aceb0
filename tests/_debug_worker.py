"""Body of the checked-build GPU test (run as a child process with B200MOE_DEBUG=1); not collected."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch
    from b200moe.ops import native
    assert native._DEBUG, "the checked library was not selected"
    lib = native.require()
    # without these symbols the range checks are not compiled in and the corrupted index below must not be launched
    assert hasattr(lib, "b2_moe_debug_read") and hasattr(lib, "b2_comm_debug_read")
    torch.manual_seed(0)
    T, D, E = 512, 256, 4
    x = torch.randn(T, D, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(E, device="cuda")[:2] for _ in range(T)]).reshape(-1)
    capacity = (2 * T + E * 255 + 255) // 256 * 256
    slot_row, row_slot, offs, tile_expert, meta, counts = native.moe_plan(idx, E, capacity)
    x_perm = native.moe_gather(x, row_slot, meta, capacity)
    weights = torch.full((T, 2), 0.5, device="cuda")
    out = native.moe_combine(x_perm, slot_row, weights.view(-1), T)
    torch.cuda.synchronize()
    assert native.debug_records() == {}
    assert float((out.float() - x.float()).abs().max()) < 1e-2      # 0.5 x + 0.5 x
    native.check_status()
    # a row index far outside the permuted buffer: the checked kernel records it and skips that token
    bad = slot_row.clone()
    bad[2 * 7] = capacity + 12345
    out2 = native.moe_combine(x_perm, bad, weights.view(-1), T)
    torch.cuda.synchronize()
    record = native.debug_records()
    assert record.get("moe", (0,))[0] == 412 and record["moe"][1] == capacity + 12345 and record["moe"][2] == capacity, record
    keep = torch.ones(T, dtype=torch.bool, device="cuda")
    keep[7] = False
    assert torch.equal(out2[keep], out[keep])
    try:
        native.check_status()
    except RuntimeError as error:
        assert "out-of-range" in str(error)
    else:
        raise AssertionError("check_status did not report the recorded violation")
    native.debug_records(clear=True)
    assert native.debug_records() == {}
    print("checked build ok")


if __name__ == "__main__":
    main()
