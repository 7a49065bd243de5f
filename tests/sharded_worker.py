"""Worker for tests/test_sharded.py: one process per rank (gloo on CPU, or nccl with one GPU each)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from tests import helpers  # noqa: E402
from torchlib_xpu_b200 import sharded, workloads  # noqa: E402


def oracle_permute(values, lengths_flat, perm):
    """The oracle's segment permutation behind the interface of sharded.kernel_permute_segments, so
    that the collective logic of distribute_inputs can run on CPU ranks (and be the checker on GPUs)."""
    out = oracle.permute_segments(values.cpu().numpy(), lengths_flat.cpu().numpy(), perm.cpu().numpy())
    return torch.from_numpy(np.ascontiguousarray(out)).to(values.device)


def checked_distribute(lengths_dp, indices_dp, weights_dp=None):
    return sharded.distribute_inputs(lengths_dp, indices_dp, weights_dp, permute=oracle_permute)


def build_problem(world):
    """The same global problem on every rank: T tables dealt round-robin, B bags."""
    T, D, B = 2 * world, 64, 8 * world
    rng = workloads.rng_for(77)
    rows = [40 + 3 * t for t in range(T)]
    W, wo, Do = helpers.float_tables(rng, rows, [D] * T, np.float16, -1, 1)
    _, offsets, indices = helpers.ragged_bags(rng, T, B, rows, 0, 9, 0.1)
    full = oracle.tbe_forward(W, oracle.FP16, wo, Do, B, indices, offsets)  # [B, T*D]
    return T, D, B, rows, W, wo, Do, offsets, indices, full


def local_problem(rank, world, T, D, B, rows, W, wo, Do, offsets, indices):
    """This rank's tables re-packed as a standalone TBE problem (table-major bags)."""
    mine = sharded.local_tables(rank, world, T)
    tabs, idx_parts, lens = [], [], []
    for g in mine:
        tabs.append(W[wo[g]:wo[g] + rows[g] * D])
        a, b = int(offsets[g * B]), int(offsets[(g + 1) * B])
        idx_parts.append(indices[a:b])
        lens.append(np.diff(offsets[g * B:(g + 1) * B + 1]))
    Wl = np.concatenate(tabs)
    wol = np.zeros(len(mine), dtype=np.int64)
    np.cumsum([t.size for t in tabs[:-1]], out=wol[1:])
    Dol = (np.arange(len(mine) + 1) * D).astype(np.int32)
    offl = np.zeros(len(mine) * B + 1, dtype=np.int64)
    np.cumsum(np.concatenate(lens), out=offl[1:])
    return mine, Wl, wol, Dol, offl, np.concatenate(idx_parts), [rows[g] for g in mine]


def expected_slice(rank, world, T, D, B, full):
    """What rank must hold after the exchange: its batch rows, columns rank-major."""
    r0, r1 = sharded.layout_batch_rows(rank, world, B)
    cols = []
    for s in range(world):
        for g in sharded.local_tables(s, world, T):
            cols.append(full[r0:r1, g * D:(g + 1) * D])
    return np.concatenate(cols, axis=1)


def check_input_distribution(rank, world, T, B, offsets, indices, offl, idxl, device, fns):
    """Every rank starts with its slice of the batch for ALL tables (the data-parallel layout) and
    must end with ALL samples for its own tables, in the bag order the lookup reads."""
    r0, r1 = sharded.layout_batch_rows(rank, world, B)
    per = r1 - r0
    lengths_dp = np.zeros((T, per), dtype=np.int64)
    parts = []
    for t in range(T):
        for bl in range(per):
            a, b = int(offsets[t * B + r0 + bl]), int(offsets[t * B + r0 + bl + 1])
            lengths_dp[t, bl] = b - a
            parts.append(indices[a:b])
    ids_dp = np.concatenate(parts).astype(np.int64) if parts else np.zeros(0, dtype=np.int64)
    w_dp = (ids_dp % 7).astype(np.float32) * 0.25
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    T_local = T // world
    for fn in fns:
        lengths_tw, offsets_tw, ids_tw, w_tw = fn(to(lengths_dp), to(ids_dp), to(w_dp))
        assert lengths_tw.shape == (T_local, B)
        np.testing.assert_array_equal(offsets_tw.cpu().numpy(), offl)
        np.testing.assert_array_equal(ids_tw.cpu().numpy(), idxl)
        np.testing.assert_array_equal(w_tw.cpu().numpy(), (idxl % 7).astype(np.float32) * 0.25)
        # without weights, and with 32-bit ids
        _, off2, ids2, none = fn(to(lengths_dp), to(ids_dp.astype(np.int32)))
        assert none is None and ids2.dtype == torch.int32
        np.testing.assert_array_equal(ids2.cpu().numpy(), idxl)
        np.testing.assert_array_equal(off2.cpu().numpy(), offl)


def main():
    backend = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group("gloo")
    T, D, B, rows, W, wo, Do, offsets, indices, full = build_problem(world)
    mine, Wl, wol, Dol, offl, idxl, rowsl = local_problem(rank, world, T, D, B, rows, W, wo, Do, offsets, indices)
    want = expected_slice(rank, world, T, D, B, full)
    local_D = len(mine) * D

    if backend == "gloo":
        check_input_distribution(rank, world, T, B, offsets, indices, offl, idxl, "cpu",
                                 [checked_distribute])
        pooled_local = torch.from_numpy(oracle.tbe_forward(Wl, oracle.FP16, wol, Dol, B, idxl, offl))
        got = sharded.reference_exchange(pooled_local)
        assert got.shape == (B // world, world * local_D)
        np.testing.assert_array_equal(got.numpy(), want)
        # gradients travel the transposed way and come back where they started
        grad_slice = torch.from_numpy(want.copy()) * (rank + 1)
        back = sharded.reference_gradient_exchange(grad_slice)
        exp = np.concatenate([full[:, g * D:(g + 1) * D] for g in mine], axis=1)
        per = B // world
        for s in range(world):
            np.testing.assert_array_equal(back[s * per:(s + 1) * per].numpy(), exp[s * per:(s + 1) * per] * (s + 1))
    else:
        from torchlib_xpu_b200 import cabi

        check_input_distribution(rank, world, T, B, offsets, indices, offl, idxl, "cuda",
                                 [checked_distribute, sharded.distribute_inputs])

        class Step:
            pass

        st = Step()
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        st.weights, st.weights_offsets, st.D_offsets = dev(Wl), dev(wol), dev(Dol)
        st.indices, st.offsets = dev(idxl), dev(offl)
        st.total_D, st.D, st.B = local_D, D, B
        ex = sharded.PooledExchange(rank, world, B, local_D)
        ex.forward_lookup(st)
        torch.cuda.synchronize()
        np.testing.assert_allclose(ex.recv.float().cpu().numpy(), want, rtol=1e-3, atol=1e-3)
        # the fused scatter and the NCCL all-to-all of the locally pooled matrix agree bit for bit
        pooled_local = cabi.forward(st.weights, st.weights_offsets, st.D_offsets, local_D, D, st.indices,
                                    st.offsets, B, output_dtype=torch.float16)
        ref = sharded.reference_exchange(pooled_local)
        assert torch.equal(ref, ex.recv)
        # gradient push == all-to-all of the gradient slices
        got = ex.gather_gradients(st).clone()
        ref_g = sharded.reference_gradient_exchange(ex.grad_slice)
        torch.cuda.synchronize()
        assert torch.equal(got, ref_g)
        # the side-stream variant: same rows once its event has fired
        ex.grad_local.zero_()
        ex.barrier()                     # no peer stores into a matrix that is still being cleared
        got2, ready = ex.gather_gradients_async(st)
        torch.cuda.current_stream().wait_event(ready)
        assert torch.equal(got2.clone(), ref_g)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("sharded worker ok (%s, world %d)" % (backend, world))


if __name__ == "__main__":
    main()
