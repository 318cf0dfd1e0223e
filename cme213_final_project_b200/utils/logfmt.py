"""The stable, regex-parsed log lines of the training driver.

Formats follow the reference field for field (``FINAL_CLEAN_CODE_/src/main.cu:229-271,420-463``) so that
log summarisers written for it keep working."""
from __future__ import annotations


def model_line(cfg) -> str:
    return (f"Model: vocab={cfg.vocab_size} seq={cfg.seq_len} hidden={cfg.hidden} heads={cfg.heads} "
            f"ff={cfg.ff} batch={cfg.batch_size}")


def params_line(count: int, elem_bytes: int = 4) -> str:
    return "Parameters: %d (%.2f KB)" % (count, count * float(elem_bytes) / 1024.0)


def training_line(epochs, lr, max_steps, world, sync_mode, overlap, bucket_kb, auto_mb) -> str:
    return ("Training: epochs=%d lr=%.2e max_steps=%d world_size=%d sync_mode=%s effective_sync=%s "
            "bucket_kb=%d auto_overlap_max_mb=%.1f"
            % (epochs, lr, max_steps, world, sync_mode, "overlap" if overlap else "blocking", bucket_kb, auto_mb))


def batches_line(total, local, used, dropped) -> str:
    return f"Batches: total={total} local_per_rank={local} used_per_epoch={used} dropped={dropped}"


def step_line(epoch, step, steps, loss) -> str:
    return "  epoch %d | step %4d/%d | loss %.4f" % (epoch, step, steps, loss)


def epoch_line(epoch, avg_loss, steps, ms, tok_s, world, overlap, start_ms, sync_ms, span) -> str:
    s = "Epoch %d: avg_logged_loss=%.4f  steps/rank=%d  %.0fms  %.0f tok/s" % (epoch, avg_loss, steps, ms, tok_s)
    if world > 1 and overlap:
        s += "  avg_grad_start=%.3fms  avg_grad_finish=%.3fms  checksum_span=%.3e" % (start_ms, sync_ms, span)
    elif world > 1:
        s += "  avg_grad_sync=%.3fms  checksum_span=%.3e" % (sync_ms, span)
    return s
