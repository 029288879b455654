"""Process-group mesh and stage manager as pure index math: a single process computes the view of every rank.
Golden tables are the expected meshes / groups / prev-next ranks of the reference's tests
(tests/test_plugins/multimodal_parallel_plugin/test_modal_process_group_mesh.py:31-57,152-178,387-396 and
test_multimodal_stage_manager.py:31-110)."""

import numpy as np
import pytest

from cornstarch_b200.parallel.mesh import MultiModalProcessGroupMesh as Mesh
from cornstarch_b200.parallel.stage_manager import MultiModalPipelineStageManager as StageManager
from cornstarch_b200.pipeline_template import PipelineTemplate


def tpl(name, stages, layers_per_stage=2):
    mods, k = [], 0
    for _ in range(stages):
        mods.append([f"layers.{k + i}" for i in range(layers_per_stage)])
        k += layers_per_stage
    return PipelineTemplate(name, mods)


ENC1, ENC2 = tpl("enc1", 2), tpl("enc2", 3)
LLM2, LLM4 = tpl("llm", 2), tpl("llm4", 4)


def test_mesh_24_ranks():
    m = Mesh({ENC1: 2}, (LLM2, 4, 1), world_size=24, rank=0)
    expected = [[[[0, 0, 1, 1]], [[2, 2, 3, 3]]], [[[4, 4, 5, 5]], [[6, 6, 7, 7]]],
                [[[8, 9, 10, 11]], [[12, 13, 14, 15]]], [[[16, 17, 18, 19]], [[20, 21, 22, 23]]]]
    assert np.array_equal(m.mesh, np.array(expected))
    assert m.modal_to_ranks[ENC1] == list(range(0, 8)) and m.modal_to_ranks[LLM2] == list(range(8, 24))
    assert m.dp_size == 2
    assert m.coords == [(0, 0, 0, 0), (0, 0, 0, 1)]


def test_mesh_40_ranks_with_sp():
    m = Mesh({ENC1: 2}, (LLM2, 4, 2), world_size=40, rank=9)
    expected = [[[[0, 0, 1, 1], [0, 0, 1, 1]], [[2, 2, 3, 3], [2, 2, 3, 3]]],
                [[[4, 4, 5, 5], [4, 4, 5, 5]], [[6, 6, 7, 7], [6, 6, 7, 7]]],
                [[[8, 9, 10, 11], [12, 13, 14, 15]], [[16, 17, 18, 19], [20, 21, 22, 23]]],
                [[[24, 25, 26, 27], [28, 29, 30, 31]], [[32, 33, 34, 35], [36, 37, 38, 39]]]]
    assert np.array_equal(m.mesh, np.array(expected))
    assert m.coords == [(2, 0, 0, 1)]


def test_groups_along_axes_24_ranks():
    m = Mesh({ENC1: 2}, (LLM2, 4, 1), world_size=24, rank=0)
    assert m.rank_sets_along_axis(Mesh.pp_axis) == [(0, 4, 8, 16), (0, 4, 9, 17), (1, 5, 10, 18), (1, 5, 11, 19),
                                                    (2, 6, 12, 20), (2, 6, 13, 21), (3, 7, 14, 22), (3, 7, 15, 23)]
    dp = m.rank_sets_along_axis(Mesh.dp_axis)
    assert dp[:3] == [(0, 2), (1, 3), (4, 6)]
    tp = m.rank_sets_along_axis(Mesh.tp_axis)
    assert (0, 1) in tp and (8, 9, 10, 11) in tp
    # an encoder rank belongs to several pipelines, one data-parallel group
    assert len(m.my_rank_sets_along_axis(Mesh.pp_axis, rank=0)) == 2
    assert m.my_rank_sets_along_axis(Mesh.dp_axis, rank=0) == [(0, 2)]


def test_world_size_must_divide():
    with pytest.raises(AssertionError):
        Mesh({ENC1: 2}, (LLM2, 4, 1), world_size=25, rank=0)


PREV_NEXT_24 = (
    [{"prev": [16, 17], "next": [4]}, {"prev": [18, 19], "next": [5]}, {"prev": [20, 21], "next": [6]}, {"prev": [22, 23], "next": [7]},
     {"prev": [0], "next": [8, 9]}, {"prev": [1], "next": [10, 11]}, {"prev": [2], "next": [12, 13]}, {"prev": [3], "next": [14, 15]},
     {"prev": [4], "next": [16]}, {"prev": [4], "next": [17]}, {"prev": [5], "next": [18]}, {"prev": [5], "next": [19]},
     {"prev": [6], "next": [20]}, {"prev": [6], "next": [21]}, {"prev": [7], "next": [22]}, {"prev": [7], "next": [23]},
     {"prev": [8], "next": [0]}, {"prev": [9], "next": [0]}, {"prev": [10], "next": [1]}, {"prev": [11], "next": [1]},
     {"prev": [12], "next": [2]}, {"prev": [13], "next": [2]}, {"prev": [14], "next": [3]}, {"prev": [15], "next": [3]}])
PREV_NEXT_18 = (
    [{"prev": [14, 15], "next": [2]}, {"prev": [16, 17], "next": [3]}, {"prev": [0], "next": [10, 11]}, {"prev": [1], "next": [12, 13]},
     {"prev": [14, 15], "next": [6]}, {"prev": [16, 17], "next": [7]}, {"prev": [4], "next": [8]}, {"prev": [5], "next": [9]},
     {"prev": [6], "next": [10, 11]}, {"prev": [7], "next": [12, 13]}, {"prev": [2, 8], "next": [14]}, {"prev": [2, 8], "next": [15]},
     {"prev": [3, 9], "next": [16]}, {"prev": [3, 9], "next": [17]}, {"prev": [10], "next": [0, 4]}, {"prev": [11], "next": [0, 4]},
     {"prev": [12], "next": [1, 5]}, {"prev": [13], "next": [1, 5]}])


@pytest.mark.parametrize("world,encs,llm,table", [
    (24, {ENC1: 2}, (LLM2, 4, 1), PREV_NEXT_24),
    (18, {ENC1: 2, ENC2: 2}, (LLM2, 4, 1), PREV_NEXT_18),
])
def test_prev_next_ranks(world, encs, llm, table):
    for rank in range(world):
        sm = StageManager(Mesh(dict(encs), llm, world_size=world, rank=rank))
        assert sm.get_prev_ranks() == table[rank]["prev"], rank
        assert sm.get_next_ranks() == table[rank]["next"], rank


def test_prev_next_84_ranks_long_chain():
    world = 84
    for rank in range(world):
        sm = StageManager(Mesh({ENC2: 4}, (LLM4, 4, 1), world_size=world, rank=rank))
        if 12 <= rank < 72:
            assert sm.get_prev_ranks() == [rank - 12] and sm.get_next_ranks() == [rank + 12]
        elif rank < 12:
            assert sm.get_prev_ranks() == [72 + rank] and sm.get_next_ranks() == [12 + rank]


def test_roles_and_layer_ranges():
    world = 24
    seen = {}
    for rank in range(world):
        m = Mesh({ENC1: 2}, (LLM2, 4, 1), world_size=world, rank=rank)
        sm = StageManager(m)
        layers = sm.distribute_layers()
        assert layers == [2, 2, 2, 2]
        seen[rank] = (sm.is_encoder, sm.stage_in_modal, sm.is_first_stage(check_only_in_modal=False),
                      sm.is_last_stage(check_only_in_modal=False), sm.get_stage_index(layers), sm.held_module_names())
    assert seen[0] == (True, 0, True, False, (0, 2), ["layers.0", "layers.1"])
    assert seen[4] == (True, 1, False, False, (2, 4), ["layers.2", "layers.3"])
    assert seen[8] == (False, 0, False, False, (0, 2), ["layers.0", "layers.1"])
    assert seen[16] == (False, 1, False, True, (2, 4), ["layers.2", "layers.3"])
    # a stage of another modality holds nothing of mine
    sm0 = StageManager(Mesh({ENC1: 2}, (LLM2, 4, 1), world_size=world, rank=0))
    assert sm0.get_stage_index([2, 2, 2, 2], stage=2) == (0, 0)
