"""Row partition of a PQ2_0 matrix over ranks (tensor parallel by output rows).

Rows are independent, so rank r of R owns rows [r * n_out / R, (r + 1) * n_out / R): a contiguous byte
range of W that starts on a 16-byte boundary whenever n_in / 128 is even.  The activation vector is
replicated; the fp32 output slices are assembled by one all-gather into y (in place: the send buffer is
the rank's own slice of the receive buffer).  No reference counterpart: the reference is single-GPU.
"""
W_BLOCK_BYTES = 34


def row_slice(n_out, rank, world):
    """Rows [lo, hi) owned by `rank`.  n_out must divide evenly (true for every model shape at 2/4/8)."""
    if n_out % world != 0:
        raise ValueError(f"n_out={n_out} does not divide over {world} ranks")
    per = n_out // world
    return rank * per, (rank + 1) * per


def byte_slice(n_out, n_in, rank, world):
    """Byte range of W (row-major PQ2_0) owned by `rank`."""
    lo, hi = row_slice(n_out, rank, world)
    row_bytes = (n_in // 128) * W_BLOCK_BYTES
    return lo * row_bytes, hi * row_bytes


def gather_rows(dist, y_full, rank, world):
    """In-place all-gather of the rank slices of y_full (a 1-D tensor of n_out floats, or [batch, n_out]
    gathered slice by slice).  `dist` is torch.distributed; works on any backend."""
    if y_full.dim() == 1:
        lo, hi = row_slice(y_full.numel(), rank, world)
        dist.all_gather_into_tensor(y_full, y_full[lo:hi])
        return y_full
    for b in range(y_full.shape[0]):
        gather_rows(dist, y_full[b], rank, world)
    return y_full
