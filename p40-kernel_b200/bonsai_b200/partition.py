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


class StepLedger:
    """Host-side record of which rank is about to launch which step of a list that spans ranks.

    The peer data plane of the list launch makes every rank wait on the device for every other rank's signal; a rank
    that never launches would leave the others to run into the device wait limit.  The ledger lets them learn it on
    the host first: before launching step s a rank writes s under its own key of a key-value store (a
    torch.distributed store: TCPStore, FileStore, or the process group's own), then asks for the ranks whose entry
    is still below s.  A rank that raised, exited or skipped its step shows up as a laggard within `timeout_s`, and
    the caller does not launch.  No reference counterpart: the reference is single-GPU.
    """

    def __init__(self, store, rank, world, prefix="bonsai_step"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def announce(self, step):
        """Say that this rank is about to launch `step` (steps count up from 1)."""
        self.store.set(self._key(self.rank), str(int(step)))

    def step_of(self, r):
        """Last step rank r announced; 0 if it never did."""
        if not self.store.check([self._key(r)]):
            return 0
        return int(self.store.get(self._key(r)).decode())

    def laggards(self, step, timeout_s=1.0, poll_s=0.01):
        """Ranks that have not announced `step` within `timeout_s`; [] when everybody is there."""
        import time
        deadline = time.monotonic() + timeout_s
        while True:
            late = [r for r in range(self.world) if self.step_of(r) < step]
            if not late or time.monotonic() >= deadline:
                return late
            time.sleep(poll_s)
