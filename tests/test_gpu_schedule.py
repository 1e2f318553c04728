"""Expert-centric scheduling against the oracle: the permutation and the segments bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import omni_oracle as orc
from _util import gen, zipf_indices

pytestmark = pytest.mark.gpu


def _check(ind: torch.Tensor, w: torch.Tensor, n: int):
    from omni_moe_b200.ops import get_scheduling_info
    s = get_scheduling_info(w.cuda(), ind.cuda(), n, 16)
    e = orc.schedule(w, ind, n)
    np.testing.assert_array_equal(s.tail_sorted_pair_ids.cpu().numpy(), e.tail_sorted_pair_ids)
    np.testing.assert_array_equal(s.tail_token_ids.cpu().numpy(), e.tail_token_ids)
    np.testing.assert_array_equal(s.tail_expert_ids.cpu().numpy(), e.tail_expert_ids)
    np.testing.assert_array_equal(s.tail_offsets.cpu().numpy(), e.tail_offsets)
    np.testing.assert_array_equal(s.tail_routing_weights.float().cpu().numpy(), e.tail_routing_weights)
    assert s.num_tail_experts == e.num_tail_experts
    assert s.max_tail_pairs_per_expert == e.max_tail_pairs_per_expert
    assert s.num_groups == 0


@pytest.mark.parametrize("t,k,n", [(64, 8, 128), (33, 6, 16), (16, 4, 4096), (1000, 16, 4096), (513, 32, 65536),
                                     (300, 64, 1 << 20), (1, 2, 7), (4096, 16, 4096), (100, 2, 3 << 20), (77, 5, 1)])
def test_schedule_uniform(t, k, n):
    g = gen(t + n)
    ind = torch.randint(0, n, (t, k), generator=g, dtype=torch.int32)
    _check(ind, torch.rand(t, k, generator=g), n)


def test_schedule_skewed_and_large_tiles():
    # Zipf(1.1): one expert owns a large share; P is large enough to take the 16-items-per-thread path
    t, k, n = 40000, 32, 262144
    ind = zipf_indices(t, k, n, 1.1, 0)
    _check(ind, torch.rand(t, k, generator=gen(1)), n)


def test_schedule_int64_and_bf16_weights():
    g = gen(9)
    ind = torch.randint(0, 1000, (200, 8), generator=g, dtype=torch.int64)
    w = torch.rand(200, 8, generator=g).bfloat16()
    from omni_moe_b200.ops import get_scheduling_info
    s = get_scheduling_info(w.cuda(), ind.cuda(), 1000, 16)
    e = orc.schedule(w, ind, 1000)
    np.testing.assert_array_equal(s.tail_sorted_pair_ids.cpu().numpy(), e.tail_sorted_pair_ids)
    np.testing.assert_array_equal(s.tail_routing_weights.float().cpu().numpy(), e.tail_routing_weights)
    assert s.tail_routing_weights.dtype == torch.bfloat16


def test_schedule_golden_reference_cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "schedule_ref.npz"))
    from omni_moe_b200.ops import get_scheduling_info
    for tag in "abc":
        w, ind, n = torch.from_numpy(g[f"{tag}.w"]), torch.from_numpy(g[f"{tag}.indices"]), int(g[f"{tag}.num_experts"])
        s = get_scheduling_info(w.cuda(), ind.cuda(), n, 16)
        np.testing.assert_array_equal(s.tail_offsets.cpu().numpy(), g[f"{tag}.tail_offsets"])
        np.testing.assert_array_equal(s.tail_expert_ids.cpu().numpy(), g[f"{tag}.tail_expert_ids"])
        assert s.max_tail_pairs_per_expert == int(g[f"{tag}.max_tail_pairs_per_expert"])
        off = g[f"{tag}.tail_offsets"]
        ref = g[f"{tag}.tail_sorted_pair_ids"]
        canon = np.concatenate([np.sort(ref[off[j]:off[j + 1]]) for j in range(len(off) - 1)])
        np.testing.assert_array_equal(s.tail_sorted_pair_ids.cpu().numpy(), canon)


def test_schedule_empty_and_bad_index():
    from omni_moe_b200.ops import get_scheduling_info, schedule
    s = get_scheduling_info(torch.zeros(0, 4).cuda(), torch.zeros(0, 4, dtype=torch.int32).cuda(), 16, 16)
    assert s.num_tail_experts == 0 and s.tail_sorted_pair_ids.numel() == 0
    ind = torch.tensor([[0, 5], [99, 1]], dtype=torch.int32).cuda()
    raw = schedule(ind, 16)
    assert raw.meta.tolist()[2] & 1  # OMNI_ST_BAD_EXPERT_INDEX, reported, nothing faults
    with pytest.raises(RuntimeError, match="expert index"):
        get_scheduling_info(torch.zeros(2, 2).cuda(), ind, 16, 16)


def test_schedule_large_table_full_size_properties():
    # 65536 tokens x 64 experts each over a 2^20-row table (4.2 M pairs): properties only
    t, k, n = 65536, 64, 1 << 20
    ind = torch.randint(0, n, (t, k), generator=gen(0), dtype=torch.int32).cuda()
    from omni_moe_b200.ops import schedule
    raw = schedule(ind, n)
    u, mx, st, _ = raw.meta.tolist()
    assert st == 0
    perm, se = raw.sorted_pair_ids.long(), raw.sorted_experts.long()
    flat = ind.flatten().long()
    assert torch.equal(flat[perm], se)                                   # keys travel with their pair ids
    assert bool((se[1:] >= se[:-1]).all())                               # sorted by expert
    same = se[1:] == se[:-1]
    assert bool((perm[1:][same] > perm[:-1][same]).all())                # stable inside an expert
    assert torch.equal(torch.sort(perm).values, torch.arange(t * k, device="cuda"))  # a permutation
    assert u == int(torch.unique(flat).numel())
    off = raw.offsets[:u + 1].long()
    assert int(off[0]) == 0 and int(off[-1]) == t * k and int((off[1:] - off[:-1]).max()) == mx
    assert torch.equal(raw.expert_ids[:u].long(), se[off[:-1]])
