"""Host-side logic of the column sharding, on CPU: the row plan, and two gloo ranks that each
compute their shard with the oracle, all-gather the slabs [ranks][rows][n_local] and rebuild the
row-major result the unsharded operator gives."""
import os
import socket

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def qi():
    module = entry.load_package()
    if not os.path.exists(module.LIB_PATH):
        module.build()
    return module


def test_shard_plan_covers_every_row_once(qi):
    for n in (3072, 9216, 12288, 18432):
        for ranks in (1, 2, 4, 8):
            rows = []
            for rank in range(ranks):
                first, count = qi.shard_plan(n, ranks, rank)
                assert count % 128 == 0 and first == rank * count
                rows.extend(range(first, first + count))
            assert rows == list(range(n))


def test_shard_plan_rejects_illegal_splits(qi):
    with pytest.raises(ValueError):
        qi.shard_plan(3072, 5, 0)       # does not divide
    with pytest.raises(ValueError):
        qi.shard_plan(512, 8, 0)        # 64 rows per rank: not a legal GEMM
    with pytest.raises(ValueError):
        qi.shard_plan(3072, 2, 2)       # rank out of range
    with pytest.raises(ValueError):
        qi.shard_plan(0, 1, 0)


def test_input_plan_keeps_whole_hadamard_blocks_and_groups(qi):
    # row-parallel split: scheme 6 slices are whole 256-input blocks, scheme 5 slices whole 64-groups
    for k, scheme, ranks in ((12288, qi.SCHEME_W4A4_H256, 8), (3072, qi.SCHEME_W4A4_H256, 4), (3072, qi.SCHEME_W4A16, 8)):
        covered = []
        for rank in range(ranks):
            first, count = qi.shard_plan_inputs(k, scheme, ranks, rank)
            assert count % (256 if scheme == qi.SCHEME_W4A4_H256 else 64) == 0 and first == rank * count
            covered.extend(range(first, first + count))
        assert covered == list(range(k))
    with pytest.raises(ValueError):
        qi.shard_plan_inputs(3072, qi.SCHEME_W4A4_H256, 8, 0)   # 384 inputs per rank cut a Hadamard block in two
    with pytest.raises(ValueError):
        qi.shard_plan_inputs(3072, 3, 2, 0)                      # not a packed scheme
    with pytest.raises(ValueError):
        qi.shard_plan_inputs(3072, qi.SCHEME_W4A16, 2, 2)


def test_placing_entry_points_reject_illegal_arguments_before_any_cuda_call(qi):
    """The argument checks of the entry points that place slices on other GPUs run on the host: they answer
    cudaErrorInvalidValue (1) without a device."""
    import ctypes
    lib = qi.lib()
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: every call below is rejected by its checks
    copies = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    invalid = 1
    scatter = lib.qi_w4a4_gemm_wide_scatter_ex
    # no copies, too many copies, a first copy out of range
    assert scatter(fake, fake, fake, fake, None, None, 2, 0, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    assert scatter(fake, fake, fake, fake, None, copies, 9, 0, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    assert scatter(fake, fake, fake, fake, None, copies, 2, 2, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    # k not a multiple of 256, a column that is not a multiple of 32, a slice that sticks out of the row
    assert scatter(fake, fake, fake, fake, None, copies, 2, 0, qi.DTYPE_F16, 512, 0, 128, 256, 384, None) == invalid
    assert scatter(fake, fake, fake, fake, None, copies, 2, 0, qi.DTYPE_F16, 512, 8, 128, 256, 256, None) == invalid
    assert scatter(fake, fake, fake, fake, None, copies, 2, 0, qi.DTYPE_F16, 256, 32, 128, 256, 256, None) == invalid
    # a copy that is not aligned for whole 32-byte sectors
    odd = (ctypes.c_void_p * 2)(0x1000, 0x2010)
    assert scatter(fake, fake, fake, fake, None, odd, 2, 0, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    # scale arrays that the CTA-pair kernel cannot stage eight bytes at a time (it is the only kernel of this entry point)
    scales_off = ctypes.c_void_p(0x1004)
    assert scatter(fake, scales_off, fake, fake, None, copies, 2, 0, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    assert scatter(fake, fake, fake, scales_off, None, copies, 2, 0, qi.DTYPE_F16, 512, 0, 128, 256, 256, None) == invalid
    # not a context
    assert lib.qi_shard_put_slice(None, copies, 2, qi.DTYPE_F16, 512, 0, 128, 256, None) == invalid
    assert lib.qi_shard_barrier(None, None) == invalid
    assert lib.qi_shard_all_reduce_f32(None, fake, 16, None) == invalid
    assert lib.qi_shard_reduce_scatter_f32(None, fake, fake, 16, None) == invalid
    offset = ctypes.c_size_t(0)
    assert lib.qi_shard_peer_export(None, ctypes.create_string_buffer(64), ctypes.byref(offset)) == invalid
    pointer = ctypes.c_void_p(0)
    assert lib.qi_shard_peer_open(None, 0, ctypes.byref(pointer)) == invalid
    assert lib.qi_shard_peer_close(None, 0) == invalid


def slabs_to_row_major(slabs: np.ndarray) -> np.ndarray:
    """[ranks, rows, n_local] -> [rows, ranks * n_local]: column block r is rank r's slice."""
    ranks, rows, n_local = slabs.shape
    return np.ascontiguousarray(slabs.transpose(1, 0, 2).reshape(rows, ranks * n_local))


def _worker(rank, ranks, port, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ranks)
    qi = entry.load_package()
    rng = np.random.default_rng(2024)  # same data on every rank
    m, n, k = 32, 512, 512
    w16 = qt.make_weights(rng, n, k)
    x16 = qt.make_activations(rng, m, k)
    first, count = qi.shard_plan(n, ranks, rank)
    outputs = {}
    # W4A4: the packer works row by row, so packing a row slice equals slicing the packed matrix
    codes, scales = qt.pack_w4a4(w16)
    shard_codes, shard_scales = qt.pack_w4a4(w16[first:first + count])
    assert np.array_equal(shard_codes, codes[first:first + count])
    assert np.array_equal(shard_scales, scales[first:first + count])
    a_codes, a_scales = qo.quantize_activations(x16)
    local = qo.w4a4_gemm(a_codes, a_scales, shard_codes, shard_scales)
    gathered = [torch.empty(m, count) for _ in range(ranks)]
    dist.all_gather(gathered, torch.from_numpy(local))
    outputs["w4a4"] = (slabs_to_row_major(torch.stack(gathered).numpy()),
                       qo.w4a4_gemm(a_codes, a_scales, codes, scales))
    codes5, scales5, minimums5 = qt.pack_w4a16(w16)
    local5 = qo.w4a16_gemm(x16, codes5[first:first + count], scales5[first:first + count],
                           minimums5[first:first + count])
    gathered5 = [torch.empty(m, count) for _ in range(ranks)]
    dist.all_gather(gathered5, torch.from_numpy(local5))
    outputs["w4a16"] = (slabs_to_row_major(torch.stack(gathered5).numpy()),
                        qo.w4a16_gemm(x16, codes5, scales5, minimums5))
    ok = all(np.array_equal(a, b) for a, b in outputs.values())
    # row-parallel: a slice of whole Hadamard blocks is quantised like the unsharded row, the partial products over
    # the ranks' input slices add up to the unsharded result (float32 rounding of the partial sums apart)
    first_k, count_k = qi.shard_plan_inputs(k, qi.SCHEME_W4A4_H256, ranks, rank)
    slice_codes, slice_scales = qo.quantize_activations(x16[:, first_k:first_k + count_k])
    ok = ok and np.array_equal(slice_codes, a_codes[:, first_k // 2:(first_k + count_k) // 2])
    ok = ok and np.array_equal(slice_scales, a_scales[:, first_k // 64:(first_k + count_k) // 64])
    partial = qo.w4a4_gemm(slice_codes, slice_scales, np.ascontiguousarray(codes[:, first_k // 2:(first_k + count_k) // 2]),
                           np.ascontiguousarray(scales[:, first_k // 64:(first_k + count_k) // 64]))
    total = torch.from_numpy(partial.copy())
    dist.all_reduce(total)
    whole = qo.w4a4_gemm(a_codes, a_scales, codes, scales)
    ok = ok and float(np.max(np.abs(total.numpy() - whole))) <= 1e-5 * float(np.max(np.abs(whole)))
    dist.barrier()
    if rank == 0:
        with open(result_path, "w") as handle:
            handle.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_gloo_ranks_rebuild_the_unsharded_result(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, port, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
