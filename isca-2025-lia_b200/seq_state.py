"""Per-sequence state for step-wise serving: one *slot* per live request.

A model registers what each of its layer runs keeps per sequence -- a *recurrent* tensor (fixed size: a matrix memory,
a normaliser, a running maximum) or a *row cache* (one row per cached token: keys/values or a compressed latent) -- and
gets back tensors whose first dimension is the slot.  Kernels address a sequence by its slot index, so a step may mix
any slots.  A slot's recurrent tensors are zeroed when it is handed out; its cached rows are simply overwritten from
position 0 (nothing past a sequence's length is ever read).  Freed slots are reused, lowest index first.

The reference keeps one static-batch KV cache per generate() call (lia/modeling_opt.py:1379-1491); requests that come and
go need this instead.
"""
import torch


class SlotError(RuntimeError):
    pass


class SlotState:
    def __init__(self, n_slots, capacity, device):
        if n_slots < 1 or capacity < 1:
            raise ValueError("n_slots and capacity must be positive")
        self.n_slots, self.capacity, self.device = int(n_slots), int(capacity), torch.device(device)
        self.recurrent = []                 # tensors [n_slots, ...] zeroed at alloc
        self.rows = []                      # tensors [n_slots, capacity, width]
        self.length = [0] * self.n_slots    # tokens each slot holds
        self.owner = [None] * self.n_slots
        self.by_id = {}

    # ---- registration (model side)
    def add_recurrent(self, shape, dtype=torch.float32):
        t = torch.zeros((self.n_slots,) + tuple(shape), dtype=dtype, device=self.device)
        self.recurrent.append(t)
        return t

    def add_rows(self, width, dtype):
        t = torch.zeros(self.n_slots, self.capacity, int(width), dtype=dtype, device=self.device)
        self.rows.append(t)
        return t

    # ---- requests (scheduler side)
    def slot_of(self, req_id):
        return self.by_id.get(req_id)

    def alloc(self, req_id):
        if req_id in self.by_id:
            raise SlotError(f"request {req_id!r} already holds slot {self.by_id[req_id]}")
        for s in range(self.n_slots):
            if self.owner[s] is None:
                self.owner[s] = req_id
                self.by_id[req_id] = s
                self.length[s] = 0
                for t in self.recurrent:
                    t[s].zero_()
                return s
        raise SlotError(f"all {self.n_slots} slots are in use")

    def free(self, req_id):
        s = self.by_id.pop(req_id, None)
        if s is None:
            raise SlotError(f"request {req_id!r} holds no slot")
        self.owner[s] = None
        self.length[s] = 0
        return s

    def reserve(self, slot, n):
        """Positions [length, length + n) of ``slot`` for the tokens of this step; returns the first."""
        p0 = self.length[slot]
        if p0 + n > self.capacity:
            raise SlotError(f"slot {slot}: {p0} + {n} tokens exceed the capacity of {self.capacity}")
        self.length[slot] = p0 + n
        return p0

    @property
    def live_tokens(self):
        return sum(self.length)
