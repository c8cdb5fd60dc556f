"""Expert-parallel plumbing on CPU: two gloo ranks run the library's EP driver
(qwen4-thor_b200/ep.py) with an oracle-backed `ops` twin; the sharded result
must equal the one-rank run of the same ops bit for bit, for even and for
heavily skewed routing (one rank receives almost everything, one nothing)."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402


class OracleOps:
    """CPU twin of ep.LibraryOps: same five steps, numpy + the C oracle."""

    def __init__(self, layer_full, lo, hi, k, world):
        self.full, self.k, self.world = layer_full, k, world
        self.E, self.hs = layer_full.E, layer_full.hs
        self.per = self.E // world
        is_, hs = layer_full.moe_is, layer_full.hs
        gb, db = O.sf_buffer_size(2 * is_, hs), O.sf_buffer_size(hs, is_)
        self.local = O.Layer(hi - lo, hs, is_, layer_full.shared_is,
                             gu_packed=layer_full.gu_packed[lo * 2 * is_:hi * 2 * is_],
                             gu_sf=layer_full.gu_sf[lo * gb:hi * gb],
                             dn_packed=layer_full.dn_packed[lo * hs:hi * hs],
                             dn_sf=layer_full.dn_sf[lo * db:hi * db],
                             gu_w_scale2=layer_full.gu_w_scale2[lo:hi], gu_input_scale=layer_full.gu_input_scale[lo:hi],
                             dn_w_scale2=layer_full.dn_w_scale2[lo:hi], dn_input_scale=layer_full.dn_input_scale[lo:hi])

    def _np(self, t):
        """bf16 rows travel as int32 pairs (gloo has no 16-bit all-to-all)."""
        if t.dtype == torch.int32 and t.dim() == 2 and t.shape[1] == self.hs // 2:
            return t.numpy().view(np.uint16).reshape(t.shape[0], self.hs)
        return t.numpy()

    def _rows(self, a_u16):
        return torch.from_numpy(np.ascontiguousarray(a_u16).view(np.int32).reshape(a_u16.shape[0], self.hs // 2).copy())

    def router(self, x):
        logits = O.bf16_linear(self._np(x), self.full.gate, 0)
        ids, rw = O.router_topk(logits, self.k)
        return torch.from_numpy(ids), torch.from_numpy(rw)

    def dispatch(self, x, ids):
        idn = ids.numpy().reshape(-1)
        dest = idn // self.per
        order = np.argsort(dest, kind="stable").astype(np.int32)
        rof = np.empty_like(order)
        rof[order] = np.arange(order.size, dtype=np.int32)
        rows = self._np(x)[order // self.k]
        counts = np.bincount(dest, minlength=self.world).astype(np.int32)
        return (self._rows(rows), torch.from_numpy((idn[order] % self.per).astype(np.int32)),
                torch.from_numpy(counts), torch.from_numpy(rof))

    def expert_rows(self, rows, local, out, n):
        if n == 0:
            return out
        ids = local.numpy().reshape(n, 1)
        _, taps = O.routed_forward(self._np(rows), ids, np.ones((n, 1), np.float32), self.local, 1, want_taps=True)
        _, _, rof, _ = O.permutation(ids, self.local.E)
        out.copy_(self._rows(taps["dn_out"][rof]))
        return out

    def finish(self, x, ret_rows, row_of_flat, rw, y):
        T = x.shape[0]
        routed = O.combine_rows(self._np(ret_rows), row_of_flat.numpy(), rw.numpy().reshape(-1), T, self.k)
        y.copy_(self._rows(O.shared_combine(self._np(x), routed, self.full, 0)))
        return y

    def empty_rows(self, n):
        return torch.empty((n, self.hs // 2), dtype=torch.int32)


def _layer(skew):
    L = synth.make_layer(E=8, hs=256, moe_is=128, shared_is=128, seed=17, per_expert_input_scale=True)
    if skew:   # push nearly every token to the experts of rank 0
        g = O.bf16_to_f32(L.gate)
        g[:4] += 0.5 * np.sign(g[:4].sum(axis=1, keepdims=True) + 1e-9)
        g[:4, 0] = 3.0
        g[4:, 0] = -3.0
        L.gate = O.f32_to_bf16(g)
    return L


def _x(T, skew):
    x = O.bf16_to_f32(synth.make_x(T, 256, seed=23))
    if skew:
        x[:, 0] = 4.0
    return torch.from_numpy(O.f32_to_bf16(x).view(np.int32).copy())


def _worker(rank, world, port, skew, T, k, out_dir):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ep = importlib.import_module("qwen4-thor_b200.ep")
    L = _layer(skew)
    per = L.E // world
    ops = OracleOps(L, rank * per, (rank + 1) * per, k, world)
    x = _x(T, skew)[rank * (T // world):(rank + 1) * (T // world)].contiguous()
    y = torch.empty_like(x)
    drv = ep.ExpertParallelMoE(ops, world, rank)
    drv.forward(x, y)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    np.save(os.path.join(out_dir, f"recv{rank}.npy"), np.array(drv.last["recv_counts"]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("skew", [False, True])
def test_two_rank_ep_equals_single_rank(tmp_path, skew):
    T, k, world = 12, 3, 2
    port = 29611 + int(skew)
    mp.spawn(_worker, args=(world, port, skew, T, k, str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    # one rank, all experts, same ops
    ep = importlib.import_module("qwen4-thor_b200.ep")
    L = _layer(skew)
    ops = OracleOps(L, 0, L.E, k, 1)
    x = _x(T, skew)
    y = torch.empty_like(x)
    ep.ExpertParallelMoE(ops, 1, 0).forward(x, y)
    assert np.array_equal(got, y.numpy())
    # and equal to the plain single-process oracle layer
    ref = O.moe_forward(x.numpy().view(np.uint16).reshape(T, 256), L, k, logits_mode=0, routed_mode=1, linear_mode=0)["y"]
    assert np.array_equal(got.view(np.uint16).reshape(T, 256), ref)
    recv = [np.load(tmp_path / f"recv{r}.npy") for r in range(world)]
    assert sum(int(r.sum()) for r in recv) == T * k
    if skew:
        assert recv[0].sum() > 3 * max(1, recv[1].sum())   # the skew really unbalances the ranks
