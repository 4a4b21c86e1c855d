"""Tensor-parallel shard algebra on the CPU: concat / sum of the oracle over shards equals the
oracle on the whole layer, and the same orchestration runs over a 2-rank gloo group."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from eptq_b200.parallel import parallel_kind, shard_activation, shard_columnwise, shard_layer, shard_rowwise
from eptq_b200.synthetic import make_activations, make_layer
from tests import util


def _W(qd, kind="e8_d4", radius=1.75):
    return oracle.dequantize_layer(util.qld_arrays(qd), util.oracle_table(kind, radius))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("qb", [None, 8])
def test_column_shards_concatenate(world, qb):
    qd = make_layer(256, 64, seed=1, outlier_frac=0.02, bias=True, qb_size=qb)
    full = _W(qd)
    parts = [_W(shard_columnwise(qd, r, world)) for r in range(world)]
    assert np.array_equal(np.concatenate(parts, axis=0), full)
    biases = torch.cat([shard_columnwise(qd, r, world).bias for r in range(world)])
    assert torch.equal(biases, qd.bias)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("qb", [None, 16])
def test_row_shards_tile_the_columns(world, qb):
    qd = make_layer(64, 256, seed=2, outlier_frac=0.02, bias=True, qb_size=qb)
    full = _W(qd)
    parts = [_W(shard_rowwise(qd, r, world)) for r in range(world)]
    assert np.array_equal(np.concatenate(parts, axis=1), full)
    x = make_activations(3, 256, seed=3)
    y_full = oracle.linear_reference(x.numpy(), full, qd.bias.numpy())
    y_sum = sum(oracle.linear_reference(shard_activation(x, r, world).numpy(), parts[r],
                                        None if shard_rowwise(qd, r, world).bias is None else qd.bias.numpy())
                for r in range(world))
    assert util.max_rel_err(y_sum, y_full) < 1e-5


def test_shard_by_name_and_errors():
    assert parallel_kind("self_attn.q_proj") == "column" and parallel_kind("mlp.down_proj") == "row"
    assert parallel_kind("fc2") == "row" and parallel_kind("lm_head") is None
    qd = make_layer(64, 64, seed=4)
    assert shard_layer(qd, "self_attn.o_proj", 1, 2).Q.shape == (8, 32)
    assert shard_layer(qd, "mlp.up_proj", 1, 2).Q.shape == (4, 64)
    assert shard_layer(qd, "something_else", 1, 2) is qd
    with pytest.raises(ValueError):
        shard_columnwise(make_layer(24, 16), 0, 2)
    with pytest.raises(ValueError):
        shard_rowwise(make_layer(16, 24), 0, 2)


def _gloo_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    qd_up = make_layer(128, 64, seed=5, outlier_frac=0.02)
    qd_down = make_layer(64, 128, seed=6, outlier_frac=0.02, bias=True)
    x = make_activations(2, 64, seed=7)
    # column-parallel up, row-parallel down, all-reduce: the MLP pattern of the decode step
    W_up = _W(shard_layer(qd_up, "mlp.up_proj", rank, world))
    hid = torch.from_numpy(oracle.linear_reference(x.numpy(), W_up)).half()      # sharded hidden
    sd = shard_layer(qd_down, "mlp.down_proj", rank, world)
    y = torch.from_numpy(oracle.linear_reference(hid.numpy(), _W(sd), None if sd.bias is None else sd.bias.numpy()))
    dist.all_reduce(y)
    if rank == 0:
        torch.save(y, out)
    dist.destroy_process_group()


def test_two_rank_gloo_mlp(tmp_path):
    port = 29500 + os.getpid() % 2000
    out = str(tmp_path / "y.pt")
    mp.spawn(_gloo_worker, args=(2, port, out), nprocs=2, join=True)
    y = torch.load(out)
    qd_up = make_layer(128, 64, seed=5, outlier_frac=0.02)
    qd_down = make_layer(64, 128, seed=6, outlier_frac=0.02, bias=True)
    x = make_activations(2, 64, seed=7)
    hid = torch.from_numpy(oracle.linear_reference(x.numpy(), _W(qd_up))).half()
    y_ref = oracle.linear_reference(hid.numpy(), _W(qd_down), qd_down.bias.numpy())
    assert util.max_rel_err(y.numpy(), y_ref) < 1e-5
