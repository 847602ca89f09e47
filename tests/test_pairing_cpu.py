"""Host-side bookkeeping that needs no GPU: the pairing of tile-dilation jobs with the launches that write their
input words (``fields.TailJob`` / ``offer_tail`` / ``take_tail``), and the split-copy requests of a first layer."""
import gc

import torch

from maskedincrementeval_b200 import fields as fl


class _Plan:
    """What a convolution plan lends a job: output geometry and the buffers the dilation fills."""

    def __init__(self, n, h, w):
        self.hout, self.wout = h, w
        nt = fl.n_tiles(n, h, w)
        self.out_bits = torch.zeros(nt, dtype=torch.int64)
        self.list = torch.zeros(nt, dtype=torch.int32)
        self.stale = torch.zeros(nt, dtype=torch.int32)
        self.counts = torch.zeros(4, dtype=torch.int32)
        self.flags = torch.zeros(nt, dtype=torch.uint8)
        self.needs_clear = False


def _fresh():
    fl.forget_tails()
    old = fl.config.tail_dilation
    fl.config.tail_dilation = True
    return old


def test_offer_take_carried_cycle():
    old = _fresh()
    try:
        bits = torch.zeros(fl.n_tiles(1, 16, 24), dtype=torch.int64)
        plan = _Plan(1, 16, 24)
        job = fl.TailJob(plan, bits, None, 1, 16, 24, 3, 1, 1)
        assert fl.take_tail(bits) is None                 # nothing offered yet; the launch is recorded as the producer
        fl.offer_tail(job)
        for _ in range(3):                                # steady state: producer carries, consumer finds it carried
            assert fl.take_tail(bits) is not None
            assert fl.tail_carried(job) and not fl.tail_carried(job)
        # the consumer sits a step out: the second take dissolves the pairing and asks for a clean start
        assert fl.take_tail(bits) is not None
        assert fl.take_tail(bits) is None and plan.needs_clear and not fl.tail_carried(job)
        assert fl.take_tail(bits) is None
    finally:
        fl.config.tail_dilation = old
        fl.forget_tails()


def test_offer_rules():
    old = _fresh()
    try:
        bits, other = torch.zeros(6, dtype=torch.int64), torch.zeros(6, dtype=torch.int64)
        plan_a, plan_b = _Plan(1, 16, 24), _Plan(1, 16, 24)
        job_a = fl.TailJob(plan_a, bits, None, 1, 16, 24, 3, 1, 1)
        fl.offer_tail(job_a)                              # input words of unknown origin: no offer
        assert fl.take_tail(bits) is None
        fl.offer_tail(job_a)
        job_b = fl.TailJob(plan_b, bits, None, 1, 16, 24, 5, 1, 2)
        fl.offer_tail(job_b)                              # the slot is taken: the second consumer keeps its own launch
        assert fl.take_tail(bits) is not None and fl.tail_carried(job_a) and not fl.tail_carried(job_b)
        # a union mask must have been written before the input's producer runs
        fl.forget_tails()
        fl.take_tail(bits)                                # producer of the input words ...
        fl.take_tail(other)                               # ... then the producer of the union words: too late
        late = fl.TailJob(plan_a, bits, other, 1, 16, 24, 3, 1, 1)
        fl.offer_tail(late)
        assert fl.take_tail(bits) is None
        fl.forget_tails()
        fl.take_tail(other)
        fl.take_tail(bits)
        fine = fl.TailJob(plan_a, bits, other, 1, 16, 24, 3, 1, 1)
        fl.offer_tail(fine)
        assert fl.take_tail(bits) is not None
        # too many tiles for one block
        fl.forget_tails()
        big_bits = torch.zeros(fl.n_tiles(2, 264, 352), dtype=torch.int64)
        fl.take_tail(big_bits)
        fl.offer_tail(fl.TailJob(_Plan(2, 264, 352), big_bits, None, 2, 264, 352, 3, 1, 1))
        assert fl.take_tail(big_bits) is None
    finally:
        fl.config.tail_dilation = old
        fl.forget_tails()


def test_offer_dies_with_the_plan_and_switch_off():
    old = _fresh()
    try:
        bits = torch.zeros(6, dtype=torch.int64)
        plan = _Plan(1, 16, 24)
        job = fl.TailJob(plan, bits, None, 1, 16, 24, 3, 1, 1)
        fl.take_tail(bits)
        fl.offer_tail(job)
        fl.config.tail_dilation = False
        assert fl.take_tail(bits) is None                 # switched off: nobody carries
        fl.config.tail_dilation = True
        assert fl.take_tail(bits) is not None and fl.tail_carried(job)
        fl.withdraw_tail(job)
        assert fl.take_tail(bits) is None
        fl.offer_tail(job)
        del plan, job                                     # the plan's buffers go away: so does the offer
        gc.collect()
        assert fl.take_tail(bits) is None
    finally:
        fl.config.tail_dilation = old
        fl.forget_tails()


def test_split_requests():
    fl.forget_tails()
    d = torch.zeros(1, 5, 16, 24)
    copy, copy_bits = torch.zeros(1, 24, 16, 24), torch.zeros(6, dtype=torch.int64)
    assert not fl.split_made(d, copy)
    fl.request_split(d, copy, copy_bits)
    assert not fl.split_made(d, copy)                     # asked, not yet made
    fl._split_requests[d.data_ptr()][2] = True            # what delta_mask does when it writes the copy
    assert fl.split_made(d, copy) and not fl.split_made(d, copy)
    assert not fl.split_made(d, torch.zeros_like(copy))   # another buffer: not this request
    fl.forget_tails()
    assert not fl._split_requests
