"""Host-side step planning of the decoder scaffold against the reference's documented example
(engine.py:262-356) and its invariants."""
import torch

from inference_engine_b200 import scaffold as S


def test_reference_example():
    # "A and B decoding, C prefilling 5 tokens, bucket 16, 5 entries: chunk_lens [1, 1, 5, 9, 0]"
    p = S.plan_step([10, 20], [(7, 5)], n_tokens=16, num_entries=5, block_m=4)
    assert p["chunk"] == [1, 1, 5, 9, 0]
    assert p["cached"] == [10, 20, 7, 0, 0]
    assert p["cu_seqlens"] == [0, 1, 2, 7, 16, 16]
    assert p["positions"] == [10, 20, 7, 8, 9, 10, 11] + list(range(9))
    assert p["seq_ids"] == [0, 1] + [2] * 5 + [3] * 9
    # every prefilling entry starts on a fresh tile, decoders get none, idle programs are -1,
    # and the tile count depends on the bucket only
    assert p["tile_start"] == [2, 6, 7, 11, 15] + [-1] * (16 // 4 + 5 - 5)
    assert p["cu_cached"] == [0, 0, 0, 7, 7, 7]
    assert p["num_decoding"] == [2]


def test_pages_disjoint_and_sufficient():
    p = S.plan_step([100, 31], [(48, 70), (0, 33)], n_tokens=128, num_entries=6, block_m=16)
    table, total = S.assign_pages(p, 16, 12, generator=torch.Generator().manual_seed(0))
    need = [(c + n + 15) // 16 for c, n in zip(p["cached"], p["chunk"])]
    used = [table[b, : need[b]].tolist() for b in range(6) if p["chunk"][b] > 0]
    flat = [x for u in used for x in u]
    assert len(flat) == len(set(flat)) == total and max(flat) == total - 1
