"""The N>1 path on CPU: two real gloo ranks exercise the amax MAX all-reduce of
sample_global_amax and the refresh/hold cadence of TrainingScaleState across ranks.
The device reduction is replaced by a host stand-in (the kernel itself is covered by the
GPU tests); the collective, the finite checks and the cadence are the real code."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, str(ROOT / "ue5m3-fp4_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ue5m3_fp4.recipe import UE5M3Recipe
        from ue5m3_fp4.scaling import training

        training._local_amax = lambda t: t.detach().float().abs().amax()
        calls = {"n": 0}
        real = dist.all_reduce

        def counting(tensor, op=None, **kw):
            calls["n"] += 1
            return real(tensor, op=op, **kw)

        dist.all_reduce = counting
        value = training.sample_global_amax(torch.tensor([float(rank + 1), -0.5]), label="unit")
        state = training.TrainingScaleState(UE5M3Recipe.proposed())
        seen = []
        for step in (1, 2, 50, 51):
            state.begin_step(step)
            local = torch.tensor([10.0 * step + rank])
            seen.append(state.reference("activation", "layers.0.mixer.up_proj", local).item())
        # all weights due at a step: one collective for the whole vector
        before = calls["n"]
        state.begin_step(60)
        sampled = state.sample_weights([(f"w{i}", torch.full((2, 2), float(10 * i + rank))) for i in range(4)])
        held = [state.reference("weight", f"w{i}", torch.zeros(2, 2)).item() for i in range(4)]
        results[rank] = (value.item(), seen, before, sampled, held, calls["n"] - before)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_share_the_global_amax_and_the_refresh_cadence():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        value, seen, collectives, sampled, held, weight_collectives = results[rank]
        assert value == 2.0  # max over ranks of (rank + 1)
        # refresh at steps 1 and 51 takes the max over ranks; steps 2 and 50 hold step 1's value
        assert seen == [11.0, 11.0, 11.0, 511.0]
        assert collectives == 3  # one direct sample + two refreshes; hold steps use no collective
        assert sampled == 4 and held == [1.0, 11.0, 21.0, 31.0] and weight_collectives == 1
