"""CPU-side checks: the C-ABI library loads and exports what include/dgpt.h declares; host logic."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "dgpt.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dgpt_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from diff_gpt_b200 import _lib

    names = _declared()
    assert len(names) >= 14
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/dgpt.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert set(_lib.PROTOTYPES) == set(names)
    assert raw.dgpt_version() == 1


def test_argument_errors_are_reported_without_a_gpu():
    from diff_gpt_b200 import _lib

    rc = _lib.lib.dgpt_embed_rmsnorm(None, None, None, 4, 8, 8, 0, None)
    assert rc == -1 and "NULL" in _lib.last_error()
    with pytest.raises(_lib.DgptError):
        _lib.check(rc)
    assert _lib.lib.dgpt_decode_attn_workspace_bytes(10, 4, 64, 1) == 0
    assert _lib.lib.dgpt_decode_attn_workspace_bytes(10, 4, 64, 3) == 10 * 4 * 3 * 66 * 4


@pytest.mark.parametrize("R,H,D,n_splits", [(3, 1, 64, 3), (1, 3, 64, 3), (5, 3, 8, 7), (1, 1, 16, 3), (7, 5, 128, 9)])
def test_split_workspace_layout_keeps_16_byte_stores_aligned(R, H, D, n_splits):
    """The accumulator block [n_splits][R*H][D] leads the workspace and D is a multiple of 4 floats, so every
    (split, row, head) accumulator starts on a 16-byte boundary whatever the parity of R*H*n_splits; the (max, sum)
    pairs follow it; the stated size covers both and is itself a multiple of 16."""
    from diff_gpt_b200 import _lib

    size = _lib.lib.dgpt_decode_attn_workspace_bytes(R, H, D, n_splits)
    slots = R * H * n_splits
    assert size % 16 == 0 and size >= slots * (D + 2) * 4
    for slot in range(slots):
        assert (slot * D * 4) % 16 == 0
    assert slots * D * 4 + slots * 2 * 4 <= size


def test_cpu_tensors_are_rejected_not_emulated():
    from diff_gpt_b200 import GPT, ops

    m = GPT(vocab_size=64, n_embd=32, block_size=16, n_head=4, n_layer=1).eval()
    with pytest.raises(RuntimeError, match="CUDA only"):
        m(torch.zeros(1, 4, dtype=torch.long))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.softcap_(torch.zeros(4), 1.0)


def test_effective_max_tokens_and_split_policy():
    from diff_gpt_b200.model.engine import _effective_max_tokens
    from diff_gpt_b200.model.gpt import _pick_splits

    assert _effective_max_tokens(16, 30, 10) == 2
    assert _effective_max_tokens(16, 32, 10) == 0
    assert _effective_max_tokens(16, 40, None) == 0
    assert _effective_max_tokens(16, 5, None) == 27
    assert _pick_splits(49152, 1280) == 1  # enough (row, head) pairs already
    assert _pick_splits(512, 4242) > 1
    assert _pick_splits(8, 100) == 1  # short: not worth a second pass


def test_paged_cache_tables_share_prompt_pages():
    from diff_gpt_b200.model.kv_cache import PagedKVCache

    c = PagedKVCache(n_layer=2, n_head=2, head_dim=8, n_series=2, rows_per_series=3, prefix_len=70, max_new=100,
                     dtype=torch.float32, device="cpu", page_tokens=64)
    assert c.prefix_pages == 2 and c.own_pages == 2 and c.suffix_slot0 == 128
    assert c.pool.shape == (2, 2 * 2 + 6 * 2, 2, 2, 64, 8)
    rt = c.row_table
    assert rt.shape == (6, 4)
    assert rt[0, :2].tolist() == rt[2, :2].tolist() == [0, 1] and rt[3, :2].tolist() == [2, 3]
    own = rt[:, 2:].reshape(-1).tolist()
    assert own == list(range(4, 16))  # contiguous per trajectory, disjoint from the prompt pages


def test_kv_cache_semantics_on_cpu_tensors():
    from diff_gpt_b200 import KVCache

    c = KVCache(batch_size=1, num_heads=1, seq_len=2, head_dim=4, num_layers=2)
    small = KVCache(batch_size=1, num_heads=1, seq_len=3, head_dim=4, num_layers=2)
    k = torch.arange(12.0).view(1, 1, 3, 4)
    c.insert_kv(0, k, -k)
    assert c.pos == 0
    kk, vv = c.insert_kv(1, k, -k)
    assert c.pos == 3 and kk.shape == (1, 1, 3, 4) and c.kv_cache.shape[4] == 2048
    assert torch.equal(vv, -k)
    other = KVCache(batch_size=4, num_heads=1, seq_len=8, head_dim=4, num_layers=2)
    with pytest.raises(AssertionError):
        KVCache(batch_size=4, num_heads=2, seq_len=8, head_dim=4, num_layers=2).prefill(c)
    small.insert_kv(0, k, -k)
    small.insert_kv(1, k, -k)
    other.prefill(small)
    assert other.pos == 3 and torch.equal(other.kv_cache[0, 0, 3, 0, :3], k[0, 0])


def test_rope_table_matches_oracle():
    from diff_gpt_b200.model.rope import apply_rotary_emb, precompute_freqs_cis
    from oracle import ref_math

    t = precompute_freqs_cis(16, 32, 10000.0)
    assert torch.allclose(t, ref_math.rope_table(16, 32), atol=1e-6)
    x = torch.randn(2, 5, 3, 16)
    assert torch.allclose(apply_rotary_emb(x, t[:5].view(1, 5, 1, 8, 2)), ref_math.rope(x, t[:5]), atol=1e-6)
