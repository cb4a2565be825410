"""MatMulId, the expert-indexed MatMul of mixture-of-experts layers (src/Sharplight.Core/Graph/StandardOps.Moe.cs:8-40):
y[t, s] = W[ids[t, s]] . x[t (, s)]. The arithmetic is the reference CPU operator's (src/Sharplight.Cpu/MatMulIdOp.cs: f32
activations against the dequantized weight), so the check is the oracle's exact product of the selected expert's
dequantized matrix at the tolerance the reference holds its f32 paths to (atol 2e-3, rtol 1e-4,
tests/Sharplight.Cpu.Tests/QuantTests.cs:257-265)."""
import numpy as np
import pytest

from helpers import FMT_OF, sl_oracle
from sharplight_b200 import native as N
from sharplight_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("type_name", ["Q4_K", "Q8_0", "Q4_0", "Q6_K", "IQ4_NL"])
@pytest.mark.parametrize("experts,n,k,tokens,slots,per_slot", [(8, 32, 512, 1, 2, False), (4, 48, 1024, 5, 3, True),
                                                               (16, 16, 256, 7, 4, False), (3, 64, 2048, 2, 1, False)])
def test_matmul_id_matches_the_selected_experts(cuda_device, type_name, experts, n, k, tokens, slots, per_slot):
    import torch
    fmt = FMT_OF[type_name]
    blocks = synth.weight_blocks(type_name, experts * n, k, seed=experts + n)
    rng = np.random.Generator(np.random.Philox(tokens * 31 + slots))
    ids = rng.integers(0, experts, (tokens, slots)).astype(np.int32)
    x = synth.activations(tokens * slots if per_slot else tokens, k + 3, seed=k)[:, :k + 3]      # rows 3 elements wider than K
    w = cuda_device.upload_weight(type_name, (experts * n, k), blocks)
    try:
        xd = torch.from_numpy(x).cuda()
        idd = torch.from_numpy(ids.reshape(-1)).cuda()
        y = torch.full((tokens * slots, n + 2), float("nan"), device="cuda")
        cuda_device.matmul_id(w, experts, xd.data_ptr(), N.F32, k + 3, idd.data_ptr(), tokens, slots, per_slot, y.data_ptr(), n + 2)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert np.all(np.isnan(got[:, n:]))                                   # nothing written beyond the N columns
        row_bytes = blocks.size // (experts * n)
        per_expert = blocks.reshape(experts, n * row_bytes)
        for t in range(tokens):
            for s in range(slots):
                item = t * slots + s
                xr = np.ascontiguousarray(x[item if per_slot else t, :k])[None, :]
                exact = sl_oracle.matmul_f64(fmt, per_expert[ids[t, s]], n, k, xr, threads=2)[0]
                assert np.all(np.abs(got[item, :n] - exact) <= 2e-3 + 1e-4 * np.abs(exact)), (t, s, int(ids[t, s]))
        assert cuda_device.last_status() == 0
        # bf16 activations
        bits = (x.view(np.uint32) >> 16).astype(np.uint16)
        xb = torch.from_numpy(bits.view(np.int16)).cuda()
        y2 = torch.zeros((tokens * slots, n), device="cuda")
        cuda_device.matmul_id(w, experts, xb.data_ptr(), N.BF16, k + 3, idd.data_ptr(), tokens, slots, per_slot, y2.data_ptr(), n)
        torch.cuda.synchronize()
        xt = (bits.astype(np.uint32) << 16).view(np.float32)
        item = tokens * slots - 1
        t, s = divmod(item, slots)
        xr = np.ascontiguousarray(xt[item if per_slot else t, :k])[None, :]
        exact = sl_oracle.matmul_f64(fmt, per_expert[ids[t, s]], n, k, xr, threads=2)[0]
        assert np.all(np.abs(y2.cpu().numpy()[item] - exact) <= 2e-3 + 1e-4 * np.abs(exact))
    finally:
        w.dispose()


def test_matmul_id_argument_checks_and_bad_ids(cuda_device):
    import torch
    experts, n, k = 4, 32, 256
    w = cuda_device.upload_weight("Q4_K", (experts * n, k), synth.weight_blocks("Q4_K", experts * n, k, seed=1))
    odd = cuda_device.upload_weight("Q4_K", (experts * 24, k), synth.weight_blocks("Q4_K", experts * 24, k, seed=2))
    q5 = cuda_device.upload_weight("Q5_K", (experts * n, k), synth.weight_blocks("Q5_K", experts * n, k, seed=3))
    try:
        x = torch.ones((2, k), device="cuda")
        ids = torch.tensor([0, 7, 1, -1], dtype=torch.int32, device="cuda")     # two ids outside [0, 4)
        y = torch.full((4, n), 5.0, device="cuda")
        with pytest.raises(Exception):
            cuda_device.matmul_id(odd, experts, x.data_ptr(), N.F32, k, ids.data_ptr(), 2, 2, False, y.data_ptr(), n)    # 24 rows per expert
        with pytest.raises(Exception):
            cuda_device.matmul_id(q5, experts, x.data_ptr(), N.F32, k, ids.data_ptr(), 2, 2, False, y.data_ptr(), n)
        with pytest.raises(Exception):
            cuda_device.matmul_id(w, 3, x.data_ptr(), N.F32, k, ids.data_ptr(), 2, 2, False, y.data_ptr(), n)            # 128 rows, 3 experts
        with pytest.raises(Exception):
            cuda_device.matmul_id(w, experts, x.data_ptr(), N.F32, k - 1, ids.data_ptr(), 2, 2, False, y.data_ptr(), n)  # stride < K
        cuda_device.matmul_id(w, experts, x.data_ptr(), N.F32, k, ids.data_ptr(), 2, 2, False, y.data_ptr(), n)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert np.all(got[1] == 5.0) and np.all(got[3] == 5.0)                   # rows of the bad ids untouched
        assert not np.any(got[0] == 5.0) and not np.any(got[2] == 5.0)
        assert cuda_device.last_status() == -1                                   # where the reference throws
    finally:
        w.dispose(); odd.dispose(); q5.dispose()
