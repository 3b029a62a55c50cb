"""Sampler-side helpers and the name-mapped weight transfer (generate/utils.py)."""
import numpy as np
import pytest
import torch

from tunix_b200.generate import utils as U


def test_small_helpers():
    assert [U.next_power_of_2(x) for x in (1, 2, 3, 9)] == [1, 2, 4, 16]
    with pytest.raises(ValueError):
        U.next_power_of_2(0)
    assert U.cdiv(9, 4) == 3
    ids = np.array([0, 0, 5, 6, 2, 0])
    assert U.find_first_non_pad_idx(ids, 0) == 2 and U.find_last_non_pad_idx(ids, 0) == 4
    assert U.find_first_eos_idx(ids, 2) == 4 and U.find_first_eos_idx(ids, [9, 6]) == 3 and U.find_first_eos_idx(ids, 7) == 6
    assert U.pad_to_length(np.array([1, 2]), 4, 9, left=True).tolist() == [9, 9, 1, 2]
    assert U.pad_to_length(torch.tensor([[1], [2]]), 3, 0, axis=0).shape == (3, 1)
    mask = torch.tensor([[0, 0, 1, 1, 1]])
    assert U.build_positions_from_mask(mask).tolist() == [[0, 0, 0, 1, 2]]
    m = U.make_causal_attn_mask(mask.bool(), cache_size=6)
    assert m.shape == (1, 5, 6) and m[0, 4].tolist() == [False, False, True, True, True, False]
    mode = [None]
    U.check_sampling_mode_conflict(mode, "greedy")
    U.check_sampling_mode_conflict(mode, "greedy")
    with pytest.raises(ValueError):
        U.check_sampling_mode_conflict(mode, "beam_search")


def test_prompt_rows():
    assert U.is_token_id_sequence([1, 2]) and U.is_token_id_sequence(np.array([1])) and not U.is_token_id_sequence("ab")
    assert not U.is_token_id_sequence([]) and not U.is_token_id_sequence(np.zeros((2, 2), np.int32))
    with pytest.raises(ValueError):
        U.as_token_ids([[1, 2]])
    assert U.unpad_prompt([0, 0, 7, 8], 2).tolist() == [7, 8] and U.unpad_prompt([0, 1], 0).size == 0
    assert U.unpad_prompt_tokens([0, 0, 7, 0, 8], pad_id=0).tolist() == [7, 0, 8]
    assert U.unpad_prompt_tokens([0, 0], pad_id=0).size == 0
    tok = lambda s: [ord(c) for c in s]  # noqa: E731
    with pytest.raises(ValueError):
        U.resolve_prompt_tokens(None, None, tok)
    with pytest.raises(ValueError):
        U.resolve_prompt_tokens("a", [[1]], tok)
    assert [r.tolist() for r in U.resolve_prompt_tokens("ab", None, tok)] == [[97, 98]]
    with pytest.raises(ValueError, match="max_model_len"):
        U.resolve_prompt_tokens(None, [[1, 2, 3]], tok, max_generation_steps=6, max_total_length=8)
    ids, lens, L = U.left_pad_prompt_tokens([[1, 2, 3, 4, 5], [6]], 4, 0, max_allowed_length=6)
    assert L == 6 and lens.tolist() == [5, 1] and ids[1].tolist() == [0, 0, 0, 0, 0, 6]
    good = [{"request_id": "a", "prompt_token_ids": [1, 2]}, {"meta_info": {"id": "b", "prompt_tokens": 1}}]
    U.check_prompt_echo([np.array([1, 2]), np.array([3])], good)
    with pytest.raises(ValueError, match="duplicate"):
        U.check_prompt_echo([np.array([1]), np.array([1])], [{"request_id": "a", "prompt_token_ids": [1]}] * 2)
    with pytest.raises(ValueError, match="differed"):
        U.check_prompt_echo([np.array([1, 2])], [{"request_id": "a", "prompt_token_ids": [1, 3]}])
    with pytest.raises(ValueError, match="count"):
        U.check_prompt_echo([np.array([1])], [])


def test_resolve_parallelism_sizes():
    assert U.resolve_parallelism_sizes(8) == (8, 1, 1)
    assert U.resolve_parallelism_sizes({"fsdp": 2, "tp": 4}, tensor_parallel_size=-1, data_parallel_size=2) == (4, 2, 1)
    assert U.resolve_parallelism_sizes((8,), 2, -1, 2) == (2, 2, 2)
    with pytest.raises(ValueError):
        U.resolve_parallelism_sizes(6, expert_parallel_size=4)


def test_transfer_with_mappings_stacked_transposed_and_aligned():
    torch.manual_seed(0)
    L, D, N, Kh, H = 3, 8, 4, 2, 2
    src = {"decoder.attn.wq": torch.randn(L, D, N, H), "decoder.attn.wk": torch.randn(L, D, Kh, H),
           "decoder.attn.k_bias": torch.randn(L, Kh * H), "embedder.table": torch.randn(11, D),
           "final_norm.scale": torch.randn(D)}
    dst = {}
    for i in range(L):
        dst[f"layers.{i}.self_attn.q_proj.weight"] = torch.zeros(N * H, D, dtype=torch.bfloat16)
        dst[f"layers.{i}.self_attn.k_proj.weight"] = torch.zeros(D, 2 * Kh, H)       # engine replicates kv heads
        dst[f"layers.{i}.self_attn.k_bias"] = torch.zeros(2 * Kh, H)
    dst["embed_tokens"] = torch.zeros(11, D)
    dst["lm_head.weight"] = torch.zeros(11, D)
    dst["norm.weight"] = torch.zeros(D)
    dst["rng.count"] = torch.zeros(1)                                                 # unmapped: left alone
    maps = {"decoder.attn.wq": ("layers.*.self_attn.q_proj.weight", ("layer", None, None, None)),
            "decoder.attn.wk": ("layers.*.self_attn.k_proj.weight", ("layer", None, None, None)),
            "decoder.attn.k_bias": ("layers.*.self_attn.k_bias", ("layer", None)),
            "embedder.table": ("embed_tokens", None), "final_norm.scale": ("norm.weight", None)}
    hooks = {"final_norm.scale": lambda v: v + 1.0}
    U.transfer_state_with_mappings(src, dst, maps, key_mapping_hook_fns=hooks, transpose_keys={"wq": (1, 2, 0)},
                                   num_kv_heads=Kh, head_dim=H)
    want_q = src["decoder.attn.wq"][1].permute(1, 2, 0).reshape(N * H, D).to(torch.bfloat16)
    assert torch.equal(dst["layers.1.self_attn.q_proj.weight"], want_q)
    k2 = dst["layers.2.self_attn.k_proj.weight"]
    assert torch.equal(k2[:, 0], src["decoder.attn.wk"][2][:, 0]) and torch.equal(k2[:, 1], k2[:, 0]) \
        and torch.equal(k2[:, 2], src["decoder.attn.wk"][2][:, 1])
    kb = dst["layers.0.self_attn.k_bias"]
    assert torch.equal(kb[0], src["decoder.attn.k_bias"][0][:H]) and torch.equal(kb[1], kb[0])
    assert torch.equal(dst["norm.weight"], src["final_norm.scale"] + 1.0)
    assert torch.equal(dst["lm_head.weight"], src["embedder.table"])                  # tied head materialised
    assert dst["rng.count"].item() == 0


def test_transfer_errors_and_chunked_reshard():
    src = {"a.w": torch.ones(4, 4), "b.w": torch.ones(2, 2)}
    dst = {"x.0.w": torch.zeros(4, 4), "x.1.w": torch.zeros(3, 3)}
    with pytest.raises(U.ShapeMismatchError):
        U.transfer_state_with_mappings(src, dst, {"a.w": ("x.0.w", None), "b.w": ("x.1.w", None)})
    with pytest.raises(U.MappingError):
        U.transfer_state_with_mappings(src, dst, {"c.w": ("x.0.w", None)})
    calls = []

    def reshard(values, specs):
        calls.append(sorted(values))
        return {k: v * 2 for k, v in values.items()}

    big = {f"p{i}": torch.full((256,), float(i)) for i in range(5)}                  # 1 KiB each
    tgt = {f"q{i}": torch.zeros(256) for i in range(5)}
    U.transfer_state_with_mappings(big, tgt, {f"p{i}": (f"q{i}", None) for i in range(5)}, reshard_fn=reshard,
                                   reshard_chunk_size=2048)
    assert [len(c) for c in calls] == [2, 2, 1] and tgt["q3"][0].item() == 6.0


def test_moe_fuse_and_interleave():
    g, u = torch.arange(8.).view(1, 8), 100 + torch.arange(8.).view(1, 8)
    plain = U.interleave_moe_weights(g, u, (1, 16), n_shards=2)
    assert plain[0].tolist() == [0, 1, 2, 3, 100, 101, 102, 103, 4, 5, 6, 7, 104, 105, 106, 107]
    lanes = U.interleave_moe_weights(g, u, (1, 16), n_shards=2, lane_size=2)
    assert lanes[0].tolist() == [0, 1, 100, 101, 2, 3, 102, 103, 4, 5, 104, 105, 6, 7, 106, 107]
    padded = U.interleave_moe_weights(g, u, (1, 24), n_shards=2)                      # per-shard width 6 > 4: zero pad
    assert padded[0, :12].tolist() == [0, 1, 2, 3, 0, 0, 100, 101, 102, 103, 0, 0]
    src = {"layers.0.moe.wi_0": torch.randn(4, 8, 6), "layers.0.moe.wi_1": torch.randn(4, 8, 6), "layers.0.moe.wo": torch.randn(4, 6, 8)}
    dst = {"layers.0.moe.wi": torch.zeros(4, 8, 12), "layers.0.moe.wo": torch.zeros(4, 6, 8)}
    fused = U.fuse_moe_weights(src, dst)
    assert set(fused) == {"layers.0.moe.wi", "layers.0.moe.wo"}
    assert torch.equal(fused["layers.0.moe.wi"][..., :6], src["layers.0.moe.wi_0"])
    assert torch.equal(fused["layers.0.moe.wi"][..., 6:], src["layers.0.moe.wi_1"])


def test_verify_state_closeness():
    a = {"w": torch.ones(3), ("l", 0, "b"): torch.zeros(2)}
    assert U.verify_state_closeness(a, {"w": torch.ones(3) + 5e-3, "l.0.b": torch.zeros(2)})
    assert not U.verify_state_closeness(a, {"w": torch.ones(3) + 0.1, "l.0.b": torch.zeros(2)})
    assert not U.verify_state_closeness(a, {"w": torch.ones(3)})
    assert not U.verify_state_closeness(a, {"w": torch.ones(4), "l.0.b": torch.zeros(2)})
