"""Column-sharded packed linears on 2 GPUs through the C ABI (NCCL all-gather over NVLink, and the W4A4
GEMM that stores its slice into every rank's output itself).
Skipped on a box with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import qipack_oracle as qo
from tests import qi_testing as qt

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _worker(rank, ranks, port, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=ranks)  # host channel for the id only
    qi = entry.load_package()
    qi.lib()
    holder = [qi.shard_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    context = qi.ShardContext(rank, ranks, holder[0])
    device = torch.device("cuda", rank)

    def up(array):
        return torch.from_numpy(np.ascontiguousarray(array)).to(device)

    rng = np.random.default_rng(99)
    m, n, k = 256, 768, 1024
    w16 = qt.make_weights(rng, n, k)
    x32 = qt.make_activations(rng, m, k).astype(np.float32)
    first, count = qi.shard_plan(n, ranks, rank)
    work = qi.LinearWork(torch.zeros(m * k // 2, dtype=torch.uint8, device=device),
                         torch.zeros(m * k // 64, dtype=torch.float16, device=device),
                         torch.zeros(m * k, dtype=torch.float16, device=device),
                         wide=torch.zeros(m * k, dtype=torch.uint8, device=device))
    ok = True
    # scheme 6, packed and byte-wide weights
    codes, scales = qt.pack_w4a4(w16)
    a_codes, a_scales = qo.quantize_activations(x32)
    expected = qo.w4a4_gemm(a_codes, a_scales, codes, scales)
    for wide in (False, True):
        shard_codes = up(codes[first:first + count])
        wide_w = None
        if wide:
            wide_w = torch.zeros(count, k, dtype=torch.uint8, device=device)
            assert qi.w4a4_widen_codes_ex(shard_codes, wide_w, count, k) == 0
        record = qi.PackedLinear(qi.SCHEME_W4A4_H256, count, k, shard_codes, up(scales[first:first + count]),
                                 weights_wide=wide_w)
        y_local = torch.zeros(m, count, dtype=torch.float32, device=device)
        y_slabs = torch.zeros(ranks, m, count, dtype=torch.float32, device=device)
        assert context.linear(record, work, up(x32), y_local, y_slabs, m) == 0
        torch.cuda.synchronize()
        assert qi.kernel_status() == 0
        rebuilt = y_slabs.cpu().numpy().transpose(1, 0, 2).reshape(m, n)
        ok = ok and np.array_equal(rebuilt, expected)
    # scheme 6 without the all-gather: every rank's GEMM stores its slice into every rank's whole output
    pool = torch.zeros(m * n * (4 + 2), dtype=torch.uint8, device=device)  # one allocation: an fp32 and an fp16 output

    def exchange(item):
        items = [None] * ranks
        dist.all_gather_object(items, item)
        return items

    peers = qi.PeerOutput(context, pool, exchange)
    a_wide = torch.zeros(m, k, dtype=torch.uint8, device=device)
    a_scales_device = torch.zeros(m, k // 64, dtype=torch.float16, device=device)
    assert qi.w4a4_quantize_activations_wide_ex(up(x32), qi.DTYPE_F32, None, a_scales_device, a_wide, m, k, None) == 0
    shard_wide = torch.zeros(count, k, dtype=torch.uint8, device=device)
    assert qi.w4a4_widen_codes_ex(up(codes[first:first + count]), shard_wide, count, k) == 0
    shard_scales = up(scales[first:first + count])
    for dtype, offset in ((qi.DTYPE_F32, 0), (qi.DTYPE_F16, m * n * 4)):
        copies = peers.copies(offset)
        assert qi.w4a4_gemm_wide_scatter_ex(a_wide, a_scales_device, shard_wide, shard_scales, None, copies,
                                            (rank + 1) % ranks, dtype, n, first, m, count, k, None) == 0
        assert context.barrier(None) == 0
    torch.cuda.synchronize()
    assert qi.kernel_status() == 0
    whole32 = pool[:m * n * 4].view(torch.float32).view(m, n).cpu().numpy()
    whole16 = pool[m * n * 4:].view(torch.float16).view(m, n).cpu().numpy()
    ok = ok and np.array_equal(whole32, expected)
    ok = ok and np.array_equal(whole16, expected.astype(np.float16))
    # the same with the slice written to this rank's own output by the ordinary GEMM and carried to the other by a copy
    dist.barrier()
    pool.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    mine = pool[m * n * 4:].view(torch.float16).view(m, n)[:, first:first + count]
    assert qi.w4a4_gemm_wide_ex(a_wide, a_scales_device, shard_wide, shard_scales, None, mine, qi.DTYPE_F16, n, m, count,
                                k, None) == 0
    assert context.put_slice(peers.copies(m * n * 4), qi.DTYPE_F16, n, first, m, count, None) == 0
    assert context.barrier(None) == 0
    torch.cuda.synchronize()
    ok = ok and np.array_equal(pool[m * n * 4:].view(torch.float16).view(m, n).cpu().numpy(), expected.astype(np.float16))
    # and with the whole output kept as slabs [ranks][rows][N/ranks]: the slice is one contiguous block
    dist.barrier()
    pool.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    slabs = pool[:ranks * m * count * 4].view(torch.float32).view(ranks, m, count)
    assert qi.w4a4_gemm_wide_ex(a_wide, a_scales_device, shard_wide, shard_scales, None, slabs[rank], qi.DTYPE_F32, count,
                                m, count, k, None) == 0
    assert context.put_slice(peers.copies(rank * m * count * 4), qi.DTYPE_F32, count, 0, m, count, None) == 0
    assert context.barrier(None) == 0
    torch.cuda.synchronize()
    ok = ok and np.array_equal(slabs.cpu().numpy().transpose(1, 0, 2).reshape(m, n), expected)
    dist.barrier()  # nobody unmaps a copy that another rank may still write
    peers.close()
    # scheme 5, fp16 output
    codes5, scales5, minimums5 = qt.pack_w4a16(w16)
    record5 = qi.PackedLinear(qi.SCHEME_W4A16, count, k, up(codes5[first:first + count]),
                              up(scales5[first:first + count]), up(minimums5[first:first + count]))
    y_local = torch.zeros(m, count, dtype=torch.float16, device=device)
    y_slabs = torch.zeros(ranks, m, count, dtype=torch.float16, device=device)
    assert context.linear(record5, work, up(x32), y_local, y_slabs, m, output_dtype=qi.DTYPE_F16) == 0
    torch.cuda.synchronize()
    expected5 = qo.w4a16_gemm(qo.f32_to_f16(x32).view(np.float16), codes5, scales5, minimums5)
    rebuilt5 = y_slabs.cpu().numpy().transpose(1, 0, 2).reshape(m, n).astype(np.float32)
    ok = ok and qt.max_relative_error(rebuilt5, expected5) <= 1e-3
    # row-parallel (K-sharded) forms: this rank's input columns of every weight row and of the activations, partial
    # products summed over the ranks (all-reduce, float32); whole Hadamard blocks / groups per slice
    for scheme in (qi.SCHEME_W4A4_H256, qi.SCHEME_W4A16):
        first_k, count_k = qi.shard_plan_inputs(k, scheme, ranks, rank)
        x_slice = np.ascontiguousarray(x32[:, first_k:first_k + count_k])
        if scheme == qi.SCHEME_W4A4_H256:
            record_k = qi.PackedLinear(scheme, n, count_k, up(codes[:, first_k // 2:(first_k + count_k) // 2]),
                                       up(scales[:, first_k // 64:(first_k + count_k) // 64]))
            whole = expected
        else:
            record_k = qi.PackedLinear(scheme, n, count_k, up(codes5[:, first_k // 2:(first_k + count_k) // 2]),
                                       up(scales5[:, first_k // 64:(first_k + count_k) // 64]),
                                       up(minimums5[:, first_k // 64:(first_k + count_k) // 64]))
            whole = expected5
        y_sum = torch.full((m, n), float("nan"), dtype=torch.float32, device=device)
        assert context.linear_inputs(record_k, work, up(x_slice), y_sum, m) == 0
        torch.cuda.synchronize()
        assert qi.kernel_status() == 0
        bound = 1e-5 if scheme == qi.SCHEME_W4A4_H256 else 1e-3
        ok = ok and qt.max_relative_error(y_sum.cpu().numpy(), whole) <= bound
    # the sum over ranks by itself
    part = torch.full((1000,), float(rank + 1), dtype=torch.float32, device=device)
    assert context.all_reduce(part, part.numel()) == 0
    torch.cuda.synchronize()
    ok = ok and bool((part == float(sum(range(1, ranks + 1)))).all())
    # and half of it: rank r keeps the r-th part of the sum
    whole = torch.arange(ranks * 500, dtype=torch.float32, device=device) * float(rank + 1)
    share = torch.full((500,), float("nan"), dtype=torch.float32, device=device)
    assert context.reduce_scatter(whole, share, 500) == 0
    torch.cuda.synchronize()
    expected_share = torch.arange(rank * 500, (rank + 1) * 500, dtype=torch.float32, device=device) * float(sum(range(1, ranks + 1)))
    ok = ok and bool((share == expected_share).all())
    assert context.destroy() == 0
    dist.barrier()
    if rank == 0:
        with open(result_path, "w") as handle:
            handle.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def test_two_ranks_all_gather_the_unsharded_result(tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, port, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
