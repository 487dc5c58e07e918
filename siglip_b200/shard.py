"""Image sharding for multi-GPU runs: the GEMM rows of different images are independent
and the weights are read-only, so every GPU takes a contiguous range of images and runs the
same kernels on its own rows with no exchange of data (the reference is single-GPU:
patch_embed.cu:104-246 has one device, one stream).
"""
from __future__ import annotations


def image_range(total_images: int, world_size: int, rank: int) -> tuple[int, int]:
    """(first image, number of images) of ``rank``: contiguous, sizes differing by at most one."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} of {world_size}")
    if total_images < 0:
        raise ValueError("negative image count")
    base, extra = divmod(total_images, world_size)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def row_range(total_images: int, rows_per_image: int, world_size: int, rank: int) -> tuple[int, int, int]:
    """(first row, number of rows, row_phase) of ``rank``.  Shards start on image boundaries, so the
    phase of the positional period is 0; it is returned for callers that split differently."""
    first, n = image_range(total_images, world_size, rank)
    return first * rows_per_image, n * rows_per_image, (first * rows_per_image) % max(rows_per_image, 1)
