"""Rank math of the parallel layout: closed-form expectations, the 9 named groups, and (when the reference is
installed next to the repository) equality with the reference for every layout up to 16 ranks."""

import itertools
import pathlib
import sys

import pytest

from fast_llm_b200.parallel.topology import DistributedConfig


def _cfg(ws, r, tp=1, pp=1, sdp=1, pf=False):
    return DistributedConfig(tensor_parallel=tp, pipeline_parallel=pp, sequence_data_parallel=sdp, pipeline_first=pf,
                             world_size=ws, rank=r, local_world_size=ws).validate()


def test_rank_formulas():
    for ws, tp, pp, sdp, pf in itertools.product((4, 8, 16), (1, 2), (1, 2), (1, 2), (False, True)):
        dp = ws // (tp * pp)
        if dp % sdp:
            continue
        for r in range(ws):
            c = _cfg(ws, r, tp, pp, sdp, pf)
            assert c.tensor_rank == r % tp
            if pf:
                assert c.pipeline_rank == (r // tp) % pp and c.data_rank == (r // tp) // pp
            else:
                assert c.data_rank == (r // tp) % dp and c.pipeline_rank == (r // tp) // dp
            assert c.sequence_data_rank == c.data_rank % sdp and c.batch_data_rank == c.data_rank // sdp
            dims = c.distributed_dims
            assert dims["world"].global_ranks == tuple(range(ws))
            for name, dim in dims.items():
                assert dim.global_ranks[dim.rank] == r and len(dim.global_ranks) == dim.size
            assert dims["tensor"].size == tp and dims["pipeline"].size == pp and dims["data"].size == dp
            assert dims["tensor_and_data"].size == tp * dp


def test_groups_partition_the_world():
    ws = 8
    for name in ("tensor", "pipeline", "data", "sequence_data", "batch_data", "tensor_and_sequence_data", "model_and_sequence_data"):
        seen = {}
        for r in range(ws):
            dim = _cfg(ws, r, tp=2, pp=2, sdp=1).distributed_dims[name]
            for member in dim.global_ranks:
                seen.setdefault(member, set()).add(dim.global_ranks)
        assert all(len(groups) == 1 for groups in seen.values()), name
    assert len(_cfg(8, 0, tp=2, pp=2).all_group_rank_sets()) > 0


def test_matches_reference_when_installed():
    ref = pathlib.Path(__file__).resolve().parent.parent / "baseline" / "_ref"
    if not (ref / "fast_llm" / "engine").is_dir():
        pytest.skip("reference not installed")
    sys.path.insert(0, str(ref))
    try:
        from fast_llm.engine.distributed.config import DistributedConfig as Ref
    except Exception as e:  # pragma: no cover
        pytest.skip(f"reference import failed: {e}")
    finally:
        sys.path.remove(str(ref))
    for ws, tp, pp, sdp, pf in itertools.product((1, 2, 4, 8), (1, 2, 4), (1, 2), (1, 2), (False, True)):
        if ws % (tp * pp) or (ws // (tp * pp)) % sdp:
            continue
        for r in range(ws):
            kw = dict(tensor_parallel=tp, pipeline_parallel=pp, sequence_data_parallel=sdp, pipeline_first=pf, world_size=ws, rank=r, local_world_size=ws)
            a, b = DistributedConfig(**kw).validate(), Ref(**kw)
            b.validate()
            for name, d in b.distributed_dims.items():
                m = a.distributed_dims[name]
                assert (m.size, m.rank, tuple(m.global_ranks)) == (d.size, d.rank, tuple(d.global_ranks)), (kw, name)
