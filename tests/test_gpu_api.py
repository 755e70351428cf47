"""The public API on a GPU replica in one process: add / pushUpdate / snapshots / stats / trace / flush / checkpoint,
and a table of tensors on the GPU."""
import pytest
import torch

import sharedtensor
from sharedtensor_b200.utils import checkpoint

pytestmark = pytest.mark.gpu


def test_gpu_master_api(free_port, tmp_path):
    torch.manual_seed(0)
    init = torch.randn(3, 4099, device="cuda")
    st = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    try:
        assert st.is_master and st.device.type == "cuda" and st.shape == init.shape
        cur = torch.empty_like(init)
        st.copyToTensor(cur)
        assert torch.equal(cur, init)
        new = cur + 0.25
        st.pushUpdate(new, cur)
        st.addFromTensor(torch.ones_like(init))
        st.copyToTensor(cur)
        assert torch.equal(cur, (init + 0.25) + 1)
        b16 = torch.empty(init.numel(), device="cuda", dtype=torch.bfloat16)
        st.copyToTensorBF16(b16)
        assert torch.equal(b16, cur.view(-1).to(torch.bfloat16))
        g = (torch.randn(init.numel(), device="cuda") * 1e-2).to(torch.bfloat16)
        st.addScaledBF16(g, -0.5)
        expect = cur.view(-1) + (-0.5) * g.float()
        st.copyToTensor(cur)
        assert torch.allclose(cur.view(-1), expect, atol=1e-6)
        with pytest.raises(ValueError, match="Not the right size!"):
            st.addFromTensor(torch.zeros(7, device="cuda"))
        with pytest.raises(ValueError):
            st.addFromTensor(torch.zeros(init.shape))  # wrong device
        s = st.stats()
        assert s["backend"] == "gpu/p2p" and s["master"] and s["device"]["errors"] == 0
        assert st.flush(5.0)
        assert st.trace() == []  # no edges, no rounds
        path = str(tmp_path / "gpu.pt")
        checkpoint.save(st, path)
        v, _ = checkpoint.load_values(path)
        assert torch.equal(v, cur.cpu())
    finally:
        st.close()


def test_gpu_table(free_port):
    tensors = {"w": torch.randn(300, 70, device="cuda") * 50, "b": torch.randn(70, device="cuda") * 1e-3}
    tab = sharedtensor.createOrFetchTable("127.0.0.1", free_port, tensors)
    try:
        assert tab.layout.offsets["b"] % 32 == 0
        tab.addFromTensors({"w": torch.ones(300, 70, device="cuda"), "b": torch.ones(70, device="cuda")})
        out = {k: torch.empty_like(v) for k, v in tensors.items()}
        tab.copyToTensors(out)
        assert torch.equal(out["w"], tensors["w"] + 1) and torch.equal(out["b"], tensors["b"] + 1)
        sc = tab.scales()
        assert sc["w"]["rms_exp"] >= 5 and sc["b"]["rms_exp"] in (-1, 0)  # the segment's zero padding counts
        flat16 = tab.new_flat(torch.bfloat16)
        tab.copyToFlatBF16(flat16)
        assert torch.equal(tab.views(flat16)["b"], out["b"].to(torch.bfloat16))
    finally:
        tab.close()
