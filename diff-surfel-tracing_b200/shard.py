"""Multi-GPU plumbing of the tracer: rays shard, surfels replicate, one all-reduce sums the gradients.

The reference is single-GPU. Rays are independent, so a multi-GPU run gives every rank a block of
rays (image rows, or whole cameras of a batch) and a full copy of the surfels and the hierarchy
(each rank runs the same deterministic build on the same vertices). The only exchange is the sum
of the per-surfel gradients after the backward trace; the binding lays all of them out in one
flat buffer, so it is a single collective.
"""
import torch
import torch.distributed as dist


def split_rows(n_rows: int, world: int, rank: int):
    """Contiguous block [start, stop) of the `n_rows` ray rows owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rays(ray_o: torch.Tensor, ray_d: torch.Tensor, world: int, rank: int):
    """This rank's rows of (H, W, 3) ray tensors (views, no copy)."""
    a, b = split_rows(ray_o.shape[0], world, rank)
    return ray_o[a:b], ray_d[a:b]


def shard_image_rows(ray_o: torch.Tensor, ray_d: torch.Tensor, world: int, rank: int, image_h: int, image_w: int, block: int = 4):
    """This rank's share of a (B, image_h * image_w, 3) batch of whole images: blocks of `block` image rows dealt
    out round-robin (rank r takes blocks r, r + world, ...) from every image, so that every rank samples every
    camera and every part of the frame (the cost of a ray depends on both). Returns contiguous (B, rows * image_w, 3)
    tensors whose rows keep their order; 4-row blocks stay whole, which is the height of the pixel tiles the
    kernels walk (pass the image width to the tracer as usual)."""
    if ray_o.dim() != 3 or ray_o.shape[1] != image_h * image_w:
        raise ValueError("expected (B, image_h * image_w, 3) ray tensors")
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank / world size")
    n_blocks = (image_h + block - 1) // block
    mine = [torch.arange(b * block, min((b + 1) * block, image_h)) for b in range(rank, n_blocks, world)]
    rows = (torch.cat(mine) if mine else torch.zeros((0,), dtype=torch.long)).to(ray_o.device)       # more ranks than row blocks: an empty share
    B = ray_o.shape[0]
    pick = lambda t: t.reshape(B, image_h, image_w, 3).index_select(1, rows).reshape(B, -1, 3).contiguous()
    return pick(ray_o), pick(ray_d)


def allreduce_bucket(bucket: torch.Tensor, group=None):
    """In-place sum of a flat gradient buffer over the ranks of `group` (no-op without a process group)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if bucket.is_cuda:
            torch.cuda.nvtx.range_push("dst_gradient_allreduce")
        dist.all_reduce(bucket, op=dist.ReduceOp.SUM, group=group)
        if bucket.is_cuda:
            torch.cuda.nvtx.range_pop()
    return bucket


def allreduce_surfel_gradients(state, group=None):
    """Sums the per-surfel gradients of the last backward call of `state` (the tracer's state object)
    over all ranks, in place and on the current stream: one collective over one flat buffer.

    For callers of the extension-level functions (`_C.trace_surfels_backward`), whose returned tensors are
    views of that buffer. Training code that goes through `SurfelTracer` and autograd should use
    `SurfelTracer.set_gradient_group()` instead: by the time `loss.backward()` returns, autograd has already
    consumed the views, and leaf gradients behind activations would stay rank-local."""
    if state.grad_bucket is None:
        raise RuntimeError("no backward call has been made on this tracer state")
    return allreduce_bucket(state.grad_bucket, group)
