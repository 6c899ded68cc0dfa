"""Distillation losses: the reference's weighted KL / reverse-KL / top-K cross-entropy loss, plain forward KL,
reverse KL and JSD, all over sparse teacher top-K targets; the fused LM-head path that never forms fp32 logits."""
from .divergence import (LOSS_KEYS, student_teacher_logprobs, loss_rows, reference_loss_segments,
                         calculate_divergence)
from .head import lmhead_stats, fused_distill_rows, distill_head_loss
