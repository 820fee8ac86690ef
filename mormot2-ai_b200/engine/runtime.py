"""What parts need to know about where and how they compute: the device, the activation
type (bfloat16, or float32 on the true 32-bit path) and which kernels are allowed."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..errors import KernelError

MAILBOX_TOKENS = 4096
MAIL_RING = 4          # copies of the mailbox that may be on their way to the host at once


class Runtime:
    def __init__(self, dtype: torch.dtype, device: str = "cuda:0", fast_kernels: bool = True,
                 guards=None):
        """``guards``: a ``cache.guards.Guards`` that the buffers of this runtime and of the
        engine built on it are made through (bands around each that a stray write damages)."""
        if dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"activations of {dtype} are not supported (bfloat16 or float32)")
        K.require_gpu()
        from ..cache.guards import alloc
        self.guards = guards
        self.dtype = dtype
        self.device = torch.device(device)
        # the tensor-core kernels serve the bfloat16 path only; the 32-bit path multiplies and
        # adds in float32 throughout
        self.fast_kernels = fast_kernels and dtype == torch.bfloat16
        # True: the tensors handed to ``bind`` belong to the engine alone, and a part that
        # re-lays a weight out (fused q/k/v, interleaved gate and up) drops the original
        self.consume_weights = False
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        # scratch of the split matrix products (float32) and the word that kernels set when
        # one of their bounded waits ran out
        self.workspace = (alloc(guards, "split-sum workspace", (16 << 20,), torch.float32,
                                self.device, None) if self.fast_kernels else None)
        # the partial sums of a split product that its consumer adds up (parts/linear.py): two
        # halves used in turn, so that two products may be pending at once (a block with two
        # branches that both defer their sums)
        self.pending_bufs = ([alloc(guards, f"pending split sums {i}", (4 << 20,), torch.float32,
                                    self.device, None) for i in range(2)]
                             if self.fast_kernels else None)
        self.pending_turn = 0
        # partial results of a decode attention whose splits are too many for one cluster
        self.attention_scratch = (alloc(guards, "attention split results", (1 << 20,),
                                        torch.float32, self.device, None)
                                  if self.fast_kernels else None)
        # word 0: set by a kernel when one of its bounded waits ran out; the words after it: the
        # tokens that the sampler chose in a step, so that one copy brings both to the host
        self.mailbox = alloc(guards, "mailbox", (1 + MAILBOX_TOKENS,), torch.int32, self.device)
        self.error_word = self.mailbox[:1]
        self.host_mailbox = torch.zeros(1 + MAILBOX_TOKENS, dtype=torch.int32).pin_memory()
        self.mail_event = torch.cuda.Event()
        # the same for steps that are read a step late (engine/decode.py)
        self.host_ring = torch.zeros((MAIL_RING, 1 + MAILBOX_TOKENS), dtype=torch.int32).pin_memory()
        self.ring_events = [torch.cuda.Event() for _ in range(MAIL_RING)]

    @property
    def pending_buf(self) -> Optional[torch.Tensor]:
        """The buffer for the next product's pending sums (the other one than last time)."""
        if self.pending_bufs is None:
            return None
        self.pending_turn ^= 1
        return self.pending_bufs[self.pending_turn]

    def check(self) -> None:
        """Raises if a kernel recorded that one of its waits ran out (synchronizes); in a debug
        build (MORMOT_B200_DEBUG=1) also if a kernel met an index outside a page table."""
        self._raise_if(int(self.error_word.item()))
        from ..csrc import build
        found = build.debug_faults()
        if found:
            raise KernelError("the kernels' index checks: " + "; ".join(found))

    def _raise_if(self, code: int) -> None:
        if code:
            self.error_word.zero_()
            raise KernelError(f"a kernel gave up a wait (code {code}: 1 load, 2 MMA, "
                              "3 epilogue; 4-5, 9-19 attention); its result is not valid")

    def token_box(self, rows: int) -> Optional[torch.Tensor]:
        """Where a sampler may leave ``rows`` chosen tokens for ``read_tokens`` (None: too many)."""
        return self.mailbox[1:1 + rows] if rows <= MAILBOX_TOKENS else None

    def read_tokens(self, rows: int) -> list:
        """The tokens in the token box and the kernels' error word in one copy through pinned
        memory (waits for the stream); raises like ``check``."""
        self.host_mailbox[:1 + rows].copy_(self.mailbox[:1 + rows], non_blocking=True)
        self.mail_event.record()
        self.mail_event.synchronize()
        got = self.host_mailbox[:1 + rows].tolist()
        self._raise_if(got[0])
        return got[1:]

    def post_mail(self, k: int, rows: int) -> None:
        """Queues a copy of the error word and the first ``rows`` tokens of the token box into
        place ``k`` of the host ring; ``take_mail(k, rows)`` waits for it."""
        self.host_ring[k, :1 + rows].copy_(self.mailbox[:1 + rows], non_blocking=True)
        self.ring_events[k].record()

    def take_mail(self, k: int, rows: int) -> list:
        self.ring_events[k].synchronize()
        got = self.host_ring[k, :1 + rows].tolist()
        self._raise_if(got[0])
        return got[1:]

    def libraries(self):
        """The kernel libraries that a model of this runtime needs."""
        libs = ["elementwise", "rope", "gemm_simt", "attention_simt", "sampling"]
        if self.fast_kernels:
            libs += ["gemm_tc", "attention_mma", "attention_tc"]
        return libs

    def attention(self, q, q_stride, out, step, line, nh, nkv, hd, window, scale) -> None:
        if self.fast_kernels:
            from ..parts import attention_fast
            if attention_fast.run(self, q, q_stride, out, step, line, nh, nkv, hd, window, scale):
                return
        K.attention_simt(q, q_stride, out, step, line, nh, nkv, hd, window, scale)
