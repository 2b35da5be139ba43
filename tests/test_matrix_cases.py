"""Equivalence and resume matrix on 8 gloo ranks (CPU, fp32).

The idea of the reference's matrix (``tests/full_stack_matrix_cases.py:209-629``, 144 cases run by
``tests/tiny_transformer_full_stack_matrix_runner.py`` in long-lived "merged" workers) with this framework's own case
list: every case is a set of ordinary training flags; ONE group of 8 worker processes builds model and runtime for case
after case through the CLI's own builders (``train.cli._build_model`` / ``_build_runtime``, i.e. the plugin selection a
user gets), trains two optimizer steps on a fixed global batch and reports the loss of every rank. The parent turns the
per-rank losses into the global loss and compares it with single-process full-batch training of the same model.

Covered: DP (sync / bucketed), ZeRO 0-3, TP, TP+SP, PP (AFAB / 1F1B), CP (all-gather K/V / zigzag ring), EP with 2 / 4 /
8-way expert groups, gradient accumulation, activation checkpointing, packed batches, LLaMA / OLMo-2 / tiny / MoE models.
The resume half (``tests/tiny_transformer_full_stack_resume.py:189-357`` in the reference) saves a sharded checkpoint
at a step boundary or in the middle of an accumulation window, rebuilds the runtime, loads and continues; the
continued losses must equal those of the uninterrupted run.
"""
import pytest
import torch

from tests.dist_utils import run_distributed

WORLD = 8
VOCAB, SEQ, GLOBAL_ROWS, STEPS = 128, 32, 8, 2

MODELS = {
    "llama": ["--model", "llama", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "4", "--hidden-size", "128", "--n-layers", "4"],
    "olmo": ["--model", "olmo2", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "4", "--hidden-size", "128", "--n-layers", "4"],
    "tiny": ["--model", "tiny", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "128", "--n-layers", "4"],
    "moe4": ["--model", "tiny_moe", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "4", "--hidden-size", "96", "--n-layers", "2", "--num-experts", "8",
             "--moe-aux-loss-coef", "0"],
    "moe": ["--model", "tiny_moe", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "96", "--n-layers", "2", "--num-experts", "8",
            "--moe-aux-loss-coef", "0"],
    # more experts than a rank has tokens: on every rank some experts get no token and therefore no gradient
    "moe64": ["--model", "tiny_moe", "--dim", "64", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "32", "--n-layers", "2", "--num-experts", "64",
              "--moe-aux-loss-coef", "0"],
}
COMMON = ["--vocab-size", str(VOCAB), "--seq-len", str(SEQ), "--lr", "1e-3", "--weight-decay", "0.01", "--grad-clip", "0.1", "--seed", "5",
          "--precision", "fp32", "--disable-metrics"]


def C(model, flags, *, accum=1, packed=False, pp_mb=None, common=""):
    """``common``: flags that change the mathematics (router, schedule) and therefore also go to the single-process baseline."""
    return dict(model=model, flags=flags.split() + common.split(), accum=accum, packed=packed, pp_mb=pp_mb, common=common)


CASES = {
    # ---- data parallel and the ZeRO stages
    "dp8_sync": C("llama", "--dp-size 8 --ddp-mode sync"),
    "dp8_async": C("llama", "--dp-size 8 --ddp-mode async"),
    "dp8_bucket_accum2": C("llama", "--dp-size 4 --tp-size 2 --use-sp --ddp-mode bucket", accum=2),
    "dp4_bucket_tp2": C("llama", "--dp-size 4 --tp-size 2 --ddp-mode bucket", accum=2),
    "dp8_zero1": C("llama", "--dp-size 8 --zero-stage 1"),
    "dp4_zero2_tp2_accum2": C("llama", "--dp-size 4 --tp-size 2 --zero-stage 2", accum=2),
    "dp8_zero3": C("llama", "--dp-size 8 --zero-stage 3"),
    "dp4_zero3_tp2_accum2": C("llama", "--dp-size 4 --tp-size 2 --zero-stage 3", accum=2),
    # ---- tensor / sequence parallel
    "dp4_tp2": C("llama", "--dp-size 4 --tp-size 2"),
    "dp4_tp2_sp": C("llama", "--dp-size 4 --tp-size 2 --use-sp"),
    "dp4_tp2_sp_zero1": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 1"),
    "dp4_tp2_sp_zero2": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 2"),
    "dp4_tp2_sp_zero3_accum2": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3", accum=2),
    "dp2_tp4_sp_zero3": C("llama", "--dp-size 2 --tp-size 4 --use-sp --zero-stage 3"),
    "tp4_dp2_sp_ckpt": C("llama", "--dp-size 2 --tp-size 4 --use-sp --activation-checkpointing"),
    "dp4_tp2_sp_zero3_ckpt": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3 --activation-checkpointing"),
    # ---- pipeline parallel
    "dp2_pp2_tp2_afab": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --pp-schedule afab", pp_mb=2),
    "dp2_pp2_tp2_1f1b_zero1": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --pp-schedule 1f1b --zero-stage 1", pp_mb=2),
    "dp2_pp2_tp2_sp_1f1b_zero2": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --use-sp --pp-schedule 1f1b --zero-stage 2", pp_mb=2),
    "dp2_pp2_tp2_sp_afab_zero3": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --use-sp --pp-schedule afab --zero-stage 3", pp_mb=2),
    "dp2_pp4_1f1b": C("llama", "--dp-size 2 --pp-size 4 --pp-schedule 1f1b", pp_mb=4),
    "dp4_pp2_afab_accum2": C("llama", "--dp-size 4 --pp-size 2 --pp-schedule afab", accum=2, pp_mb=1),
    # ---- context parallel
    "dp2_pp2_cp2_allgather_afab": C("llama", "--dp-size 2 --pp-size 2 --cp-size 2 --cp-attn-core all_gather_kv --pp-schedule afab", pp_mb=2),
    "dp2_pp2_cp2_ring_1f1b_zero1": C("llama", "--dp-size 2 --pp-size 2 --cp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag "
                                              "--pp-schedule 1f1b --zero-stage 1", pp_mb=2),
    "dp2_cp2_tp2_sp_ring_zero3": C("llama", "--dp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag --zero-stage 3"),
    "dp2_cp2_tp2_allgather_zero2": C("llama", "--dp-size 2 --cp-size 2 --tp-size 2 --cp-attn-core all_gather_kv --zero-stage 2"),
    "pp2_cp2_tp2_sp_ring_1f1b": C("llama", "--pp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag --pp-schedule 1f1b",
                                  pp_mb=2),
    "pp2_cp2_tp2_allgather_afab": C("llama", "--pp-size 2 --cp-size 2 --tp-size 2 --cp-attn-core all_gather_kv --pp-schedule afab", pp_mb=4),
    "dp2_cp4_ring_zero1": C("llama", "--dp-size 2 --cp-size 4 --cp-attn-core ring --cp-token-planner fixed_zigzag --zero-stage 1"),
    "dp4_bucket_cp2_ring": C("llama", "--dp-size 4 --cp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --ddp-mode bucket", accum=2),
    "dp4_cp2_ring_contiguous": C("llama", "--dp-size 4 --cp-size 2 --cp-attn-core ring --cp-token-planner fixed_contiguous"),
    # ---- packed rows (several documents per row, padding at the end)
    "packed_dp4_tp2_sp_zero3": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3", packed=True),
    "packed_dp4_tp2_sp": C("llama", "--dp-size 4 --tp-size 2 --use-sp", packed=True),
    "packed_dp4_tp2_zero3": C("llama", "--dp-size 4 --tp-size 2 --zero-stage 3", packed=True),
    "packed_dp8_zero1": C("llama", "--dp-size 8 --zero-stage 1", packed=True),
    "packed_dp2_cp2_tp2_ring": C("llama", "--dp-size 2 --cp-size 2 --tp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag", packed=True),
    "packed_dp4_pp2_1f1b": C("llama", "--dp-size 4 --pp-size 2 --pp-schedule 1f1b", packed=True, pp_mb=2),
    "packed_dp4_cp2_allgather_zero2": C("llama", "--dp-size 4 --cp-size 2 --cp-attn-core all_gather_kv --zero-stage 2", packed=True),
    # ---- OLMo-2 (post-norm, QK-norm over the sharded projection width)
    "olmo_dp4_tp2": C("olmo", "--dp-size 4 --tp-size 2"),
    "olmo_dp4_tp2_sp_zero3": C("olmo", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3"),
    "olmo_dp4_tp2_sp_zero3_ckpt": C("olmo", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3 --activation-checkpointing", accum=2),
    "olmo_dp2_pp2_tp2_1f1b": C("olmo", "--dp-size 2 --pp-size 2 --tp-size 2 --pp-schedule 1f1b", pp_mb=2),
    "olmo_packed_dp2_cp2_tp2_ring": C("olmo", "--dp-size 2 --cp-size 2 --tp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag", packed=True),
    "olmo_dp8_zero1": C("olmo", "--dp-size 8 --zero-stage 1"),
    # the 13B packed recipe at toy size: TP2 x CP2 (zigzag ring) x PP2, 1F1B with 8 micro-batches, SP, activation checkpointing
    "olmo_packed_pp2_cp2_tp2_sp_ring_1f1b_ckpt": C("olmo", "--pp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag "
                                                           "--pp-schedule 1f1b --activation-checkpointing", packed=True, pp_mb=8),
    # packed rows do not split their targets evenly over context-parallel ranks: every pipeline micro-batch needs its own loss weight
    "olmo_packed_dp2_cp2_tp2_sp_ring": C("olmo", "--dp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag", packed=True),
    "olmo_packed_dp2_pp2_cp2_ring_1f1b": C("olmo", "--dp-size 2 --pp-size 2 --cp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --pp-schedule 1f1b", packed=True, pp_mb=4),
    "packed_pp2_cp2_tp2_sp_ring_1f1b": C("llama", "--pp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag --pp-schedule 1f1b", packed=True, pp_mb=8),
    "packed_dp2_cp2_tp2_sp_allgather": C("llama", "--dp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core all_gather_kv", packed=True),
    # ---- expert parallel (expert groups of 8, 4 and 2 ranks inside the data-parallel axis)
    "moe_dp8_ep8": C("moe", "--dp-size 8 --ep-size 8"),
    "moe_dp8_ep4_zero2": C("moe", "--dp-size 8 --ep-size 4 --zero-stage 2"),
    "moe_dp8_ep2_zero1": C("moe", "--dp-size 8 --ep-size 2 --zero-stage 1"),
    "moe_dp4_tp2_ep4": C("moe", "--dp-size 4 --tp-size 2 --ep-size 4"),
    "moe_dp4_pp2_ep2_1f1b": C("moe", "--dp-size 4 --pp-size 2 --ep-size 2 --pp-schedule 1f1b", pp_mb=2),
    "moe_dp4_pp2_ep4_afab_zero2": C("moe", "--dp-size 4 --pp-size 2 --ep-size 4 --pp-schedule afab --zero-stage 2", pp_mb=1, accum=2),
    "moe_dp8_ep1_zero3": C("moe", "--dp-size 8 --zero-stage 3"),
    # ---- reduced precision (master weights in fp32; compared with the fp32 baseline at bf16 tolerance)
    "bf16_dp4_tp2_sp_zero3": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3 --precision bf16"),
    "bf16_dp4_tp2_zero1_accum2": C("llama", "--dp-size 4 --tp-size 2 --zero-stage 1 --precision bf16", accum=2),
    "bf16_dp2_pp2_tp2_1f1b": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --pp-schedule 1f1b --precision bf16", pp_mb=2),
    "fp16_dp8_zero2": C("llama", "--dp-size 8 --zero-stage 2 --precision fp16"),
    # ---- further combinations
    "moe_dp8_ep4_zero3": C("moe", "--dp-size 8 --ep-size 4 --zero-stage 3"),
    "moe_dp4_cp2_ep4_ring": C("moe", "--dp-size 4 --cp-size 2 --ep-size 4 --cp-attn-core ring --cp-token-planner fixed_zigzag"),
    "tiny_dp2_pp2_cp2_ring_1f1b": C("tiny", "--dp-size 2 --pp-size 2 --cp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --pp-schedule 1f1b", pp_mb=2),
    "olmo_dp2_pp2_cp2_allgather_zero1": C("olmo", "--dp-size 2 --pp-size 2 --cp-size 2 --cp-attn-core all_gather_kv --zero-stage 1", pp_mb=2),
    "packed_dp2_pp2_tp2_sp_1f1b_zero3": C("llama", "--dp-size 2 --pp-size 2 --tp-size 2 --use-sp --pp-schedule 1f1b --zero-stage 3", packed=True, pp_mb=2),
    "packed_moe_dp4_tp2_ep4_zero2": C("moe", "--dp-size 4 --tp-size 2 --ep-size 4 --zero-stage 2", packed=True),
    "dp2_tp4_sp_zero1_accum2": C("llama", "--dp-size 2 --tp-size 4 --use-sp --zero-stage 1", accum=2),
    "pp4_tp2_sp_1f1b": C("llama", "--pp-size 4 --tp-size 2 --use-sp --pp-schedule 1f1b", pp_mb=4),
    "pp4_dp2_afab_zero2": C("llama", "--pp-size 4 --dp-size 2 --pp-schedule afab --zero-stage 2", pp_mb=2),
    "cp8_ring": C("llama", "--cp-size 8 --cp-attn-core ring --cp-token-planner fixed_zigzag"),
    "cp8_allgather_packed": C("llama", "--cp-size 8 --cp-attn-core all_gather_kv", packed=True),
    "packed_dp2_cp2_pp2_allgather_zero2": C("llama", "--dp-size 2 --cp-size 2 --pp-size 2 --cp-attn-core all_gather_kv --zero-stage 2 --pp-schedule 1f1b",
                                            packed=True, pp_mb=2),
    "moe_dp8_ep8_zero1": C("moe", "--dp-size 8 --ep-size 8 --zero-stage 1"),
    "olmo_pp2_cp2_tp2_ring_afab": C("olmo", "--pp-size 2 --cp-size 2 --tp-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --pp-schedule afab", pp_mb=4),
    "dp8_async_ckpt": C("llama", "--dp-size 8 --ddp-mode async --activation-checkpointing"),
    "tiny_dp2_cp2_tp2_sp_ring_zero2": C("tiny", "--dp-size 2 --cp-size 2 --tp-size 2 --use-sp --cp-attn-core ring --cp-token-planner fixed_zigzag --zero-stage 2"),
    # ---- choices that change the mathematics: the baseline gets them too
    "moe_top2_dp8_ep4": C("moe", "--dp-size 8 --ep-size 4", common="--moe-top-k 2"),
    "moe_top2_dp4_tp2_ep2_zero1": C("moe", "--dp-size 4 --tp-size 2 --ep-size 2 --zero-stage 1", common="--moe-top-k 2"),
    "cosine_dp4_tp2_sp_zero3": C("llama", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3", common="--lr-schedule cosine --warmup-steps 1 --max-steps 6"),
    "ckpt_every2_dp4_tp2_sp": C("llama", "--dp-size 4 --tp-size 2 --use-sp --activation-checkpointing --activation-checkpoint-every-n-layers 2"),
    # expert group reusing the tensor-parallel ranks under sequence parallelism: every TP rank holds different experts and different tokens
    "moe_dp4_tp2_sp_ep4": C("moe", "--dp-size 4 --tp-size 2 --use-sp --ep-size 4"),
    "moe_dp4_tp2_sp_ep2": C("moe", "--dp-size 4 --tp-size 2 --use-sp --ep-size 2"),
    "moe_top2_dp4_tp2_sp_ep2_zero2": C("moe", "--dp-size 4 --tp-size 2 --use-sp --ep-size 2 --zero-stage 2", common="--moe-top-k 2"),
    "moe_dp2_pp2_tp2_sp_ep2_1f1b": C("moe", "--dp-size 2 --pp-size 2 --tp-size 2 --use-sp --ep-size 2 --pp-schedule 1f1b", pp_mb=2),
    "moe_dp2_cp2_tp2_sp_ep2_ring_zero1": C("moe", "--dp-size 2 --cp-size 2 --tp-size 2 --use-sp --ep-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --zero-stage 1"),
    "moe_dp2_cp2_tp2_ep2_allgather": C("moe", "--dp-size 2 --cp-size 2 --tp-size 2 --ep-size 2 --cp-attn-core all_gather_kv"),
    "moe_top2_dp2_cp4_ep2_ring_zero3": C("moe", "--dp-size 2 --cp-size 4 --ep-size 2 --cp-attn-core ring --cp-token-planner fixed_zigzag --zero-stage 3", common="--moe-top-k 2"),
    "moe_dp2_tp4_ep2": C("moe4", "--dp-size 2 --tp-size 4 --ep-size 2"),
    "moe_dp2_tp4_sp_ep2_zero1": C("moe4", "--dp-size 2 --tp-size 4 --use-sp --ep-size 2 --zero-stage 1"),
    "moe64_dp4_tp2_bucket_accum2": C("moe64", "--dp-size 4 --tp-size 2 --ddp-mode bucket", accum=2),
    "moe64_dp8_async": C("moe64", "--dp-size 8 --ddp-mode async"),
    "moe64_dp8_zero3": C("moe64", "--dp-size 8 --zero-stage 3"),
    "moe64_dp4_tp2_sp_ep4_zero2_accum2": C("moe64", "--dp-size 4 --tp-size 2 --use-sp --ep-size 4 --zero-stage 2", accum=2),
    "moe_dp4_tp2_sp": C("moe", "--dp-size 4 --tp-size 2 --use-sp"),
    "moe_dp4_tp2": C("moe", "--dp-size 4 --tp-size 2"),
    # load-balance loss switched on: it is a statistic of the LOCAL batch, so these are compared with each other (same data
    # sharding, experts placed differently), not with the full-batch baseline
    "moe_aux_dp8": C("moe", "--dp-size 8", common="--moe-aux-loss-coef 0.05"),
    "moe_aux_dp8_ep4": C("moe", "--dp-size 8 --ep-size 4", common="--moe-aux-loss-coef 0.05"),
    "moe_aux_dp8_ep8_zero2": C("moe", "--dp-size 8 --ep-size 8 --zero-stage 2", common="--moe-aux-loss-coef 0.05"),
    # context parallelism cuts every sequence in two: the balance term of a rank covers half the tokens and is weighted 1 / cp
    "moe_aux_dp4_cp2": C("moe", "--dp-size 4 --cp-size 2", common="--moe-aux-loss-coef 0.05"),
    "moe_aux_dp4_cp2_ring_ep4": C("moe", "--dp-size 4 --cp-size 2 --cp-attn-core ring --ep-size 4", common="--moe-aux-loss-coef 0.05"),
    "moe_aux_dp4_tp2": C("moe", "--dp-size 4 --tp-size 2", common="--moe-aux-loss-coef 0.05"),
    "moe_aux_dp4_pp2": C("moe", "--dp-size 4 --pp-size 2 --pp-schedule 1f1b", common="--moe-aux-loss-coef 0.05", pp_mb=1),
    "moe_aux_dp4_pp2_ep4": C("moe", "--dp-size 4 --pp-size 2 --ep-size 4 --pp-schedule 1f1b", common="--moe-aux-loss-coef 0.05", pp_mb=1),
    # capacity-limited top-2 routing drops assignments per LOCAL batch: compared across expert placements as well
    "moe_aux_cap_dp8": C("moe", "--dp-size 8", common="--moe-top-k 2 --moe-capacity-factor 0.75 --moe-aux-loss-coef 0.05"),
    "moe_aux_cap_dp8_ep4_zero1": C("moe", "--dp-size 8 --ep-size 4 --zero-stage 1", common="--moe-top-k 2 --moe-capacity-factor 0.75 --moe-aux-loss-coef 0.05"),
    "moe_aux_cap_dp4_tp2_sp_ep4": C("moe", "--dp-size 4 --tp-size 2 --use-sp --ep-size 4", common="--moe-top-k 2 --moe-capacity-factor 0.75 --moe-aux-loss-coef 0.05"),
    "moe_aux_cap_dp4_tp2_sp": C("moe", "--dp-size 4 --tp-size 2 --use-sp", common="--moe-top-k 2 --moe-capacity-factor 0.75 --moe-aux-loss-coef 0.05"),
    "bf16_dp8": C("llama", "--dp-size 8 --precision bf16"),
    "bf16_dp8_zero1": C("llama", "--dp-size 8 --zero-stage 1 --precision bf16"),
    "bf16_dp8_zero3": C("llama", "--dp-size 8 --zero-stage 3 --precision bf16"),
    # ---- the small reference transformer
    "tiny_dp4_tp2_sp_zero3": C("tiny", "--dp-size 4 --tp-size 2 --use-sp --zero-stage 3"),
    "tiny_dp4_pp2_afab": C("tiny", "--dp-size 4 --pp-size 2 --pp-schedule afab", pp_mb=2),
}

RESUME = {   # case name -> micro-steps to run before the checkpoint (a multiple of the case's accumulation = step boundary)
    "dp4_tp2_sp_zero3_accum2": 2, "dp4_zero3_tp2_accum2": 3, "dp2_pp2_tp2_1f1b_zero1": 1, "dp2_cp2_tp2_sp_ring_zero3": 1, "moe_dp8_ep4_zero2": 1,
    "olmo_dp4_tp2_sp_zero3_ckpt": 3, "dp2_pp2_tp2_sp_afab_zero3": 1,
    # bf16 with fp32 master weights: the masters, not the rounded model weights, must come back
    "bf16_dp4_tp2_sp_zero3": 1, "bf16_dp4_tp2_zero1_accum2": 3, "fp16_dp8_zero2": 1, "bf16_dp8": 1, "bf16_dp8_zero1": 1, "bf16_dp8_zero3": 1,
    "cosine_dp4_tp2_sp_zero3": 1, "bf16_dp2_pp2_tp2_1f1b": 1, "moe_top2_dp8_ep4": 1,
    "dp4_pp2_afab_accum2": 1, "moe_dp4_pp2_ep2_1f1b": 1, "packed_dp2_cp2_tp2_ring": 1, "moe_dp8_ep4_zero3": 1,
    # in the middle of an accumulation window WITHOUT a sharded optimizer: the partial gradients travel with the checkpoint
    "dp4_bucket_tp2": 3, "dp8_bucket_accum2": 1,
    "moe_dp4_tp2_sp_ep4": 1, "cp8_ring": 1, "olmo_packed_pp2_cp2_tp2_sp_ring_1f1b_ckpt": 1, "moe_top2_dp2_cp4_ep2_ring_zero3": 1,
}


def _global_batches(packed: bool):
    """[step] -> dict of [GLOBAL_ROWS, SEQ] tensors, identical in every process."""
    g = torch.Generator().manual_seed(77 + int(packed))
    out = []
    for _ in range(STEPS + 1):
        ids = torch.randint(0, VOCAB, (GLOBAL_ROWS, SEQ), generator=g)
        batch = {"input_ids": ids, "labels": ids.roll(-1, 1).clone()}
        if packed:
            seq = torch.full((GLOBAL_ROWS, SEQ), -1, dtype=torch.long)
            pos = torch.zeros((GLOBAL_ROWS, SEQ), dtype=torch.long)
            for r in range(GLOBAL_ROWS):
                cuts = sorted({0, int(torch.randint(6, 14, (1,), generator=g)), int(torch.randint(16, 26, (1,), generator=g)), SEQ - 3})
                for d, (a, b) in enumerate(zip(cuts, cuts[1:])):
                    seq[r, a:b] = d
                    pos[r, a:b] = torch.arange(b - a)
                    batch["labels"][r, b - 1] = -100           # the last token of a document has no target
            batch["labels"][seq == -1] = -100
            batch["sequence_ids"], batch["position_ids"] = seq, pos
        out.append(batch)
    return out


def _args(case):
    import maltos_b200  # noqa: F401
    from maltos_b200.train import flags

    argv = MODELS[case["model"]] + COMMON + case["flags"] + ["--grad-accum-steps", str(case["accum"])]
    if case["pp_mb"]:
        argv += ["--pp-microbatches", str(case["pp_mb"])]
    a = flags.parse_args_from(argv + ["--micro-batch-size", "1"], require_data=False)
    a.micro_batch_size = GLOBAL_ROWS // (a.dp_size * case["accum"])
    return a


def _micro_batch(batch, dp_rank, dp, accum, m):
    rows = GLOBAL_ROWS // (dp * accum)
    assert rows >= 1, "the case leaves no row for a micro-step"
    lo = (m * dp + dp_rank) * rows
    return {k: v[lo:lo + rows].clone() for k, v in batch.items()}


def _build(case):
    from maltos_b200.train import cli

    a = _args(case)
    cli.validate_args(a, WORLD)
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    return a, core


def _worker(rank, world, names):
    import torch.distributed as dist

    from maltos_b200.runtime.mesh import MeshAxis

    results = {}
    for name in names:
        case = CASES[name]
        try:
            a, core = _build(case)
            core.setup()
            core.model.train()
            dp_group = core.get_group(MeshAxis.DP)
            dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
            losses, norms = [], []
            for step in range(STEPS):
                for m in range(case["accum"]):
                    loss, should = core.run_step(_micro_batch(_global_batches(case["packed"])[step], dp_rank, a.dp_size, case["accum"], m))
                assert should
                core.step_optimizer()
                metrics = core.collect_metrics()
                losses.append(float(metrics["loss"]))      # mean over the accumulation window
                norms.append(next((float(v) for k, v in metrics.items() if k.endswith("/grad_norm")), None))
            spread = _replica_spread(core)
            core.close()
            results[name] = ("ok", losses, a.cp_size, spread, norms)
        except Exception as exc:  # noqa: BLE001 - one broken case must not hide the others
            import traceback

            results[name] = ("error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}", 1, 0.0)
            try:
                dist.barrier()
            except Exception:
                pass
    return results


def _replica_spread(core) -> float:
    """Largest difference between the copies of a parameter held by the ranks that replicate it, over every mesh axis the
    checkpoint metadata declares it replicated on (data / context parallel ranks; tensor parallel ranks for norms and
    other unsharded weights). Must be exactly zero: every replica applies the same update to the same reduced gradient - a
    nonzero value means two gradient reductions raced or one was skipped."""
    import torch.distributed as dist

    from maltos_b200.runtime.mesh import MeshAxis
    from maltos_b200.runtime.types import ParamRole

    worst = 0.0
    for name, entry in core.state_manager.params.items():
        p = entry.param
        if p.untyped_storage().size() == 0:
            continue        # ZeRO-3 parameters are not materialised between steps
        axes = set(entry.attrs.replicated_axes)
        if core.get_param_role(p) == ParamRole.EXPERT:
            axes &= {MeshAxis.EREP}          # an expert's copies live on the expert-replica group only
        if axes & {MeshAxis.DP, MeshAxis.CP, MeshAxis.DCP}:
            axes = (axes - {MeshAxis.DP, MeshAxis.CP}) | {MeshAxis.DCP}
        for axis in sorted(axes, key=lambda a: a.value):
            if axis not in (MeshAxis.DCP, MeshAxis.TP, MeshAxis.EREP):
                continue
            group = core.get_group(axis)
            if group is None or dist.get_world_size(group) <= 1:
                continue
            lo, hi = p.detach().float().clone(), p.detach().float().clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
            worst = max(worst, float((hi - lo).abs().max()))
    return worst


def _baseline(model: str, packed: bool, common: str = ""):
    """Single process, the whole global batch as one micro-batch."""
    from maltos_b200.train import cli

    case = C(model, "--dp-size 1", common=common)
    a = _args(case)
    a.micro_batch_size = GLOBAL_ROWS
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    core.model.train()
    losses, norms = [], []
    for step in range(STEPS):
        loss, _ = core.run_step({k: v.clone() for k, v in _global_batches(packed)[step].items()})
        core.step_optimizer()
        losses.append(float(loss.detach()))
        norms.append(next((float(v) for k, v in core.collect_metrics().items() if k.endswith("/grad_norm")), None))
    core.close()
    return losses, norms


CHUNK = 10   # cases per group of worker processes: a case that fails takes only its own chunk down


@pytest.fixture(scope="module")
def matrix_results():
    names = sorted(CASES)
    merged = [dict() for _ in range(WORLD)]
    for i in range(0, len(names), CHUNK):
        chunk = names[i:i + CHUNK]
        try:
            part = run_distributed(_worker, WORLD, chunk, timeout=420.0)
        except BaseException as exc:  # noqa: BLE001 - reported per case below
            part = [{n: ("error", f"worker group failed: {type(exc).__name__}: {str(exc)[:1500]}", 1, 0.0) for n in chunk} for _ in range(WORLD)]
        for r in range(WORLD):
            merged[r].update(part[r])
    return merged


@pytest.fixture(scope="module")
def baselines():
    return {key: _baseline(*key) for key in sorted({(c["model"], c["packed"], c["common"]) for c in CASES.values()})}


def test_case_list_is_wide_enough():
    assert len(CASES) >= 40
    flags = " ".join(" ".join(c["flags"]) for c in CASES.values())
    for needle in ("--zero-stage 1", "--zero-stage 2", "--zero-stage 3", "--pp-schedule 1f1b", "--pp-schedule afab", "--cp-attn-core ring",
                   "--cp-attn-core all_gather_kv", "--ep-size 8", "--ep-size 4", "--ep-size 2", "--use-sp", "--activation-checkpointing",
                   "--ddp-mode bucket"):
        assert needle in flags, needle
    assert {c["model"] for c in CASES.values()} == set(MODELS) and any(c["packed"] for c in CASES.values())


AUX_PAIRS = [("moe_aux_dp8", "moe_aux_dp8_ep4"), ("moe_aux_dp8", "moe_aux_dp8_ep8_zero2"), ("moe_aux_dp4_pp2", "moe_aux_dp4_pp2_ep4"),
             ("moe_aux_cap_dp8", "moe_aux_cap_dp8_ep4_zero1"), ("moe_aux_cap_dp4_tp2_sp", "moe_aux_cap_dp4_tp2_sp_ep4")]


@pytest.mark.parametrize("plain,expert_parallel", AUX_PAIRS)
def test_load_balance_loss_is_the_same_wherever_the_experts_live(plain, expert_parallel, matrix_results):
    """With the auxiliary loss on, expert parallelism (and ZeRO on top) must not change loss or gradient norm of a run
    with the same data sharding."""
    for step in range(STEPS):
        vals = []
        for name in (plain, expert_parallel):
            per_rank = [r[name] for r in matrix_results]
            for status, payload, *_ in per_rank:
                assert status == "ok", payload
            vals.append((sum(r[1][step] for r in per_rank) / WORLD, per_rank[0][4][step]))
        (la, na), (lb, nb) = vals
        assert abs(la - lb) < 2e-5 and (na is None or nb is None or abs(na - nb) < 2e-5 * max(1.0, na)), (step, vals)


@pytest.mark.parametrize("cp_case", ["moe_aux_dp4_cp2", "moe_aux_dp4_cp2_ring_ep4"])
def test_load_balance_loss_has_the_same_strength_under_context_parallelism(cp_case, matrix_results):
    """The balance term is a product of two token averages, so halves of a sequence do not give exactly the value of the
    whole - but nearly; counted once per context-parallel rank (gradients are summed over that group) it would be off by
    the whole term (~0.05 here). Compared with a run whose data-parallel ranks see the same rows uncut."""
    for step in range(STEPS):
        vals = []
        for name in ("moe_aux_dp4_tp2", cp_case):
            per_rank = [r[name] for r in matrix_results]
            for status, payload, *_ in per_rank:
                assert status == "ok", payload
            vals.append((sum(r[1][step] for r in per_rank) / WORLD, per_rank[0][4][step]))    # the logged loss is cp x the share
        (la, na), (lb, nb) = vals
        assert abs(la - lb) < 4e-3, (step, vals)
        assert na is None or nb is None or abs(na - nb) < 0.03 * na, (step, vals)


@pytest.mark.parametrize("name", sorted(n for n in CASES if not n.startswith("moe_aux_")))
def test_case_matches_single_process_training(name, matrix_results, baselines):
    case = CASES[name]
    per_rank = [r[name] for r in matrix_results]
    for status, payload, *_ in per_rank:
        assert status == "ok", payload
    assert max(r[3] for r in per_rank) == 0.0, (name, "replicas of shared parameters drifted apart", [r[3] for r in per_rank])
    cp = per_rank[0][2]
    ref, ref_norms = baselines[(case["model"], case["packed"], case["common"])]
    for step in range(STEPS):
        # the clipped norm is the norm of the GLOBAL gradient: every rank must report the single-process value (AdamW hides a
        # wrong clip coefficient from the loss, so the norm is checked directly)
        for r in per_rank:
            if r[4][step] is not None and "--precision" not in case["flags"]:
                assert abs(r[4][step] - ref_norms[step]) < 2e-5 * max(1.0, ref_norms[step]), (name, step, r[4][step], ref_norms[step])
        # every rank reports the loss of its data shard (context-parallel ranks: cp x their share), so the plain mean is global
        got = sum(r[1][step] for r in per_rank) / WORLD
        tol = 2e-5                       # fp32: only the order of summation differs from the single process
        if "--precision" in case["flags"]:
            tol = 2e-3                   # bf16 / fp16 compute against the fp32 baseline
        assert abs(got - ref[step]) < tol, (name, step, got, ref[step])


# ------------------------------------------------------------------------------------------------ resume
def _resume_worker(rank, world, names, root):
    import os

    import torch.distributed as dist

    from maltos_b200.runtime.mesh import MeshAxis
    from maltos_b200.state import save_sharded_checkpoint

    results = {}
    for name in names:
        case, stop_after = CASES[name], RESUME[name]
        try:
            total_micro = (STEPS + 1) * case["accum"]

            def run(core, a, first, last, dp_rank):
                out = []
                for i in range(first, last):
                    step, m = divmod(i, case["accum"])
                    loss, should = core.run_step(_micro_batch(_global_batches(case["packed"])[step], dp_rank, a.dp_size, case["accum"], m))
                    out.append(float(loss.detach()))
                    if should:
                        core.step_optimizer()
                return out

            def fresh():
                a, core = _build(case)
                return a, core

            a, core = fresh()
            core.setup()
            core.model.train()
            dp_group = core.get_group(MeshAxis.DP)
            dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
            continuous = run(core, a, 0, total_micro, dp_rank)
            core.close()

            a, core = fresh()
            core.setup()
            core.model.train()
            head = run(core, a, 0, stop_after, dp_rank)
            ckpt = os.path.join(root, name, "step_00000001")
            save_sharded_checkpoint(core.state_manager, ckpt)
            core.close()

            a, core = fresh()
            core.setup(checkpoint_path=ckpt)
            core.model.train()
            tail = run(core, a, stop_after, total_micro, dp_rank)
            core.close()
            results[name] = ("ok", continuous, head + tail)
        except Exception as exc:  # noqa: BLE001
            import traceback

            results[name] = ("error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-1500:]}", None)
            try:
                dist.barrier()
            except Exception:
                pass
    return results


@pytest.fixture(scope="module")
def resume_results(tmp_path_factory):
    root = tmp_path_factory.mktemp("matrix_resume")
    names = sorted(RESUME)
    merged = [dict() for _ in range(WORLD)]
    for i in range(0, len(names), 4):
        chunk = names[i:i + 4]
        try:
            part = run_distributed(_resume_worker, WORLD, chunk, str(root), timeout=420.0)
        except BaseException as exc:  # noqa: BLE001
            part = [{n: ("error", f"worker group failed: {type(exc).__name__}: {str(exc)[:1500]}", None) for n in chunk} for _ in range(WORLD)]
        for r in range(WORLD):
            merged[r].update(part[r])
    return merged


@pytest.mark.parametrize("name", sorted(RESUME))
def test_resume_equals_uninterrupted_training(name, resume_results):
    """Checkpoint at a step boundary or in the middle of an accumulation window, rebuild, load, continue."""
    mid = RESUME[name] % CASES[name]["accum"] != 0
    for rank, res in enumerate(resume_results):
        status, continuous, resumed = res[name]
        assert status == "ok", continuous
        assert len(continuous) == len(resumed)
        worst = max(abs(x - y) for x, y in zip(continuous, resumed))
        # partial gradients travel with a checkpoint taken inside an accumulation window (sharded or not), master weights come
        # back in fp32: the continuation is the same computation
        limit = 5e-5
        assert worst < limit, (name, rank, mid, continuous, resumed)
