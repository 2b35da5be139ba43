"""Variable-length attention helpers on CPU: layout metadata, pack/unpack, fallback equivalence."""
import torch

from maltos_b200.ops.attention import attention_reference
from maltos_b200.runtime.layers import flash_utils as fu
from maltos_b200.utils.constants import PAD_SEQUENCE_ID


def _ids():
    seq = torch.full((2, 12), PAD_SEQUENCE_ID, dtype=torch.long)
    seq[0, :5], seq[0, 5:9] = 0, 1
    seq[1, :3], seq[1, 3:12] = 0, 0     # two rows never join, even with equal ids
    seq[1, 3:12] = 1
    return seq


def test_varlen_metadata_and_roundtrip():
    seq = _ids()
    meta = fu._varlen_qkv_metadata(seq)
    assert meta.cu_seqlens.tolist() == [0, 5, 9, 12, 21] and meta.max_seqlen == 9
    assert fu._varlen_qkv_metadata(seq) is meta            # cached on the tensor
    seq[0, 8] = PAD_SEQUENCE_ID                            # in-place change invalidates the cache
    assert fu._varlen_qkv_metadata(seq).cu_seqlens.tolist() == [0, 5, 8, 11, 20]
    q = torch.randn(2, 12, 4, 8)
    packed = fu.pack_varlen_qkv(q, q[:, :, :2], q[:, :, :2], seq)
    assert packed.q.shape == (20, 4, 8) and packed.k.shape == (20, 2, 8)
    back = fu.unpack_varlen_output_by_indices(packed.q, packed.flat_indices, batch_size=2, seq_len=12)
    mask = (seq != PAD_SEQUENCE_ID).unsqueeze(-1).unsqueeze(-1)
    assert torch.equal(back, q * mask)
    empty = torch.full((1, 4), PAD_SEQUENCE_ID, dtype=torch.long)
    assert fu._varlen_qkv_metadata(empty).max_seqlen == 0


def test_varlen_fallback_matches_reference_and_segments_agree():
    torch.manual_seed(0)
    seq = _ids()
    q, k, v = torch.randn(2, 12, 4, 8), torch.randn(2, 12, 2, 8), torch.randn(2, 12, 2, 8)
    assert fu.flash_attn_fallback_reason(q) is not None      # CPU fp32: the library's masked attention runs
    out = fu.flash_attn_varlen(q, k, v, seq)
    order = torch.arange(12).unsqueeze(0).expand(2, 12)
    ref = attention_reference(q, k, v, q_positions=order, k_positions=order, q_sequence_ids=seq, k_sequence_ids=seq)
    mask = (seq != PAD_SEQUENCE_ID).unsqueeze(-1).unsqueeze(-1)
    assert torch.allclose(out, ref * mask, atol=1e-5)
    meta = fu._varlen_qkv_metadata(seq)
    seg = fu.flash_attn_varlen_segments(q, k, v, token_indices=meta.flat_indices, cu_seqlens=meta.cu_seqlens, max_seqlen=meta.max_seqlen)
    assert torch.allclose(seg, out, atol=1e-5)
    blk = fu.flash_attn_dense_with_lse(q, k, v, q_positions=order, k_positions=order)
    assert blk.out.shape == q.shape and blk.lse.shape == (2, 4, 12)
