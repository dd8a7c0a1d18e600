"""A pack file end to end on the GPU: written, verified, opened, its data section uploaded verbatim, each record
handed to the dispatcher as the view qi_pack_linear builds (what transformer.cplus:569-572 and :673-713 do per
call), and the outputs compared with the oracle on the weights that went in."""
import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("scheme,policy", [(6, "transformer:w4a4-h256-g64-v6"), (5, "transformer:w4a16-g64-v6")])
def test_linears_run_straight_from_an_uploaded_pack(tmp_path, scheme, policy):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    qi = entry.load_package()
    qi.lib()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(900 + scheme)
    shapes = [(384, 256), (256, 768), (640, 512)]
    tensors = [{"name": "norm.weight", "scheme": 1, "dimensions": [256], "weights": np.ones(256, dtype=np.float16)}]
    stored = []
    for index, (n, k) in enumerate(shapes):
        w16 = qt.make_weights(rng, n, k)
        if scheme == 6:
            codes, scales = qt.pack_w4a4(w16)
            tensors.append({"name": f"blocks.{index}.weight", "scheme": 6, "dimensions": [n, k], "group_size": 64,
                            "weights": codes, "scales": scales})
            stored.append((codes, scales, None))
        else:
            codes, scales, minimums = qt.pack_w4a16(w16)
            tensors.append({"name": f"blocks.{index}.weight", "scheme": 5, "dimensions": [n, k], "group_size": 64,
                            "weights": codes, "scales": scales, "zeros": minimums})
            stored.append((codes, scales, minimums))
    path = str(tmp_path / "model.qipack")
    qi.pack_write(path, policy, tensors, metadata="steps=4\n")
    assert qi.pack_verify(path, len(tensors), len(shapes)) == 0
    pack = qi.Pack(path)
    try:
        resident = torch.from_numpy(pack.data()).cuda()  # the data section, verbatim
        rows = 200
        for index, (n, k) in enumerate(shapes):
            with pytest.raises(qi.PackError):
                pack.linear(0, resident)  # the vector is not a packed linear
            record = pack.linear(index + 1, resident)
            assert (record.scheme, record.n, record.k) == (scheme, n, k)
            x32 = qt.make_activations(rng, rows, k).astype(np.float32)
            work = qi.LinearWork(torch.zeros(rows * k // 2, dtype=torch.uint8, device="cuda"),
                                 torch.zeros(rows * k // 64, dtype=torch.float16, device="cuda"),
                                 torch.zeros(rows * k, dtype=torch.float16, device="cuda"))
            y = torch.full((rows, n), float("nan"), dtype=torch.float32, device="cuda")
            assert qi.linear(record, work, torch.from_numpy(x32).cuda(), y, rows) == 0
            torch.cuda.synchronize()
            assert qi.kernel_status() == 0
            codes, scales, minimums = stored[index]
            if scheme == 6:
                a_codes, a_scales = qo.quantize_activations(x32)
                assert np.array_equal(y.cpu().numpy(), qo.w4a4_gemm(a_codes, a_scales, codes, scales))
            else:
                expected = qo.w4a16_gemm(qo.f32_to_f16(x32).view(np.float16), codes, scales, minimums)
                assert qt.max_relative_error(y.cpu().numpy(), expected) <= 1e-3
    finally:
        pack.close()
