"""Test infrastructure only: a Python restatement of the reference's allocator policy (core/soliton/alloc.d), used
to check the product's C++ pool counter by counter on random traces. Nothing in the product imports this.

Restated line by line from alloc.d: roundSize :54-60, mix :62-66, rawAlloc :68-86 (limit check against reserved),
arenaAlloc :98-111, alloc :128-174 (exact-size cache scanned front to back, swap-remove; one flush-and-retry),
release :176-200, releaseArena :204-213, emptyCache :215-223; and the stats / reset of api.d:143-164.
Addresses are modelled as tokens, one per raw block: the test checks that the library hands the cached blocks out in
the same order as this model does.
"""
MASK = (1 << 64) - 1
FNV_SEED, FNV_PRIME = 1469598103934665603, 1099511628211


def round_size(n):
    small, large = 512, 2 << 20
    n = max(n, 1)
    return (n + small - 1) // small * small if n < (1 << 20) else (n + large - 1) // large * large


class PoolModel:
    def __init__(self):
        self.cache = []          # [(size, token)] in the reference's array order
        self.allocated = self.reserved = self.peak_allocated = self.peak_reserved = 0
        self.n_alloc = self.n_raw = 0
        self.limit = 0
        self.hash = FNV_SEED
        self.next_token = 1

    def _mix(self, kind, n):
        self.hash = ((self.hash ^ kind) * FNV_PRIME) & MASK
        self.hash = ((self.hash ^ n) * FNV_PRIME) & MASK

    def _raw_alloc(self, n):
        if self.limit and self.reserved + n > self.limit:
            return None
        self.next_token += 1
        return self.next_token

    def empty_cache(self):
        for size, _ in self.cache:
            self.reserved -= size
        self.cache = []

    def alloc(self, n):
        n = round_size(n)
        self._mix(1, n)
        token = None
        for i, (size, tok) in enumerate(self.cache):
            if size == n:
                token = tok
                self.cache[i] = self.cache[-1]
                self.cache.pop()
                break
        if token is None:
            token = self._raw_alloc(n)
            if token is None:
                self.empty_cache()
                token = self._raw_alloc(n)
            if token is None:
                return None
            self.reserved += n
            self.n_raw += 1
            self.peak_reserved = max(self.peak_reserved, self.reserved)
        self.allocated += n
        self.n_alloc += 1
        self.peak_allocated = max(self.peak_allocated, self.allocated)
        return token

    def release(self, token, n):
        n = round_size(n)
        self._mix(2, n)
        self.allocated -= n
        self.cache.append((n, token))

    def reset_stats(self):
        self.peak_allocated, self.peak_reserved = self.allocated, self.reserved
        self.n_alloc = self.n_raw = 0
        self.hash = FNV_SEED

    def stats(self):
        h = self.hash if self.hash < (1 << 63) else self.hash - (1 << 64)  # the C ABI returns it as a signed long
        return [self.allocated, self.reserved, self.peak_allocated, self.peak_reserved, self.n_alloc, self.n_raw, h]
