"""Frame-level data parallelism: which frames a rank owns and how per-rank times become one number.

The reference is single-GPU and batch 1 (se-ssd-ai-trt.cpp:1723, :1125). Frames never need data from
other frames, so N GPUs run N independent shards with no collective on the data path; the process group
only carries a barrier and the maximum over ranks of the device time.
"""
from __future__ import annotations

from . import synth


def first_frame(rank: int, frames_per_rank: int) -> int:
    """Index of the first frame of `rank`'s shard (weak scaling: every rank has frames_per_rank frames)."""
    return rank * frames_per_rank


def frame_seed(frame_index: int) -> int:
    """Seed of frame `frame_index` of the throughput sweep."""
    return synth.SEED_BASE + 5 + 1000 * (frame_index + 1)


def job_throughput(elapsed_ms, frames_per_rank: int, steps: int, world: int, all_reduce_max=None) -> float:
    """frames/s of the whole job: all ranks' frames over the slowest rank's time.

    elapsed_ms: 1-element tensor holding this rank's device milliseconds; all_reduce_max reduces it in
    place over the ranks (None for a single process).
    """
    if all_reduce_max is not None and world > 1:
        all_reduce_max(elapsed_ms)
    return frames_per_rank * steps * world / (float(elapsed_ms[0]) / 1e3)
