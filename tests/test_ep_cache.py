"""Cache bookkeeping; mirrors what the reference's tests/test_ep_cache.py pins
(put/get/contains, byte accounting, send-buffer collection after completion,
a random-operation soak against a list model) on CPU tensors."""
import random

import pytest
import torch

from dice_b200.expertpara.ep_cache import All2AllCache, EPSkipCache


class DummyHandle:
    def __init__(self, completed=True):
        self.completed = completed
        self.waited = False

    def is_completed(self):
        return self.completed

    def wait(self):
        self.waited = True
        self.completed = True


def _nbytes(t):
    return t.element_size() * t.numel()


def test_put_get_contains_and_sizes():
    cache = All2AllCache(capacity=10, val_len=3, gc_send_buf=False)
    assert cache.tensors_size() == 0
    t1, t2 = torch.randn(10, 10), torch.randn(5, 5)
    cache.put(1, (None, t1, None))
    assert cache.contains(1) and not cache.contains(0)
    assert cache.tensors_size() == _nbytes(t1)
    cache.put(5, (None, t2, t1))
    assert cache.tensors_size() == 2 * _nbytes(t1) + _nbytes(t2)
    assert cache.get(5)[1] is t2 and cache.contains(5)  # get does not remove
    cache.clear()
    assert cache.tensors_size() == 0 and not cache.contains(1)


def test_value_shape_is_enforced():
    cache = All2AllCache(capacity=2, val_len=3, gc_send_buf=False)
    with pytest.raises(AssertionError):
        cache.put(0, (None, torch.zeros(1)))
    with pytest.raises(AssertionError):
        cache.put(0, ("not a list", torch.zeros(1), None))
    with pytest.raises(AssertionError):
        cache.put(0, (None, torch.zeros(1), "not a tensor"))


def test_send_buffer_collected_only_after_completion():
    cache = All2AllCache(capacity=4, val_len=3, gc_send_buf=True)
    h = DummyHandle(completed=False)
    recv, send = torch.randn(4, 4), torch.randn(8, 8)
    cache.put(0, ([h], recv, send))
    cache.put(1, (None, torch.randn(2), None))  # triggers a collection pass: handle still busy
    assert cache.get(0)[-1] is send and cache.get(0)[0] == [h]
    h.completed = True
    cache.put(2, (None, torch.randn(2), None))
    assert cache.get(0)[-1] is None and cache.get(0)[0] is None and cache.get(0)[1] is recv
    # the byte accounting follows the collection
    assert cache.tensors_size() == _nbytes(recv) + 2 * _nbytes(torch.randn(2))


def test_recv_buffer_collection_is_manual_and_opt_in():
    off = All2AllCache(capacity=2, val_len=3, gc_send_buf=False, gc_recv_buf=False)
    off.put(0, (None, torch.randn(3), None))
    off.manual_gc_recv_buf()
    assert off.cache[0][1] is not None
    on = All2AllCache(capacity=2, val_len=3, gc_send_buf=False, gc_recv_buf=True)
    busy = DummyHandle(False)
    on.put(0, ([busy], torch.randn(3), None))
    on.put(1, (None, torch.randn(3), None))
    on.manual_gc_recv_buf()
    assert on.cache[0][1] is not None and on.cache[1][1] is None


def test_wait_waits_for_every_handle():
    cache = All2AllCache(capacity=3, val_len=3, gc_send_buf=False)
    hs = [DummyHandle(False) for _ in range(3)]
    cache.put(0, ([hs[0], hs[1]], torch.zeros(1), None))
    cache.put(2, ([hs[2]], torch.zeros(1), None))
    cache.wait()
    assert all(h.waited for h in hs)


def test_random_operations_against_a_list_model():
    random.seed(42)
    cap = 6
    cache = All2AllCache(capacity=cap, val_len=4, gc_send_buf=False)
    model = [None] * cap
    for _ in range(1000):
        op = random.choice(["put", "get", "contains", "clear", "size"])
        key = random.randrange(cap)
        if op == "put":
            val = (None, torch.randn(random.randint(1, 9)), random.random(), None)
            cache.put(key, val)
            model[key] = val
        elif op == "get" and model[key] is not None:
            assert cache.get(key) is model[key]
        elif op == "contains":
            assert cache.contains(key) == (model[key] is not None)
        elif op == "clear" and random.random() < 0.05:
            cache.clear()
            model = [None] * cap
        elif op == "size":
            assert cache.tensors_size() == sum(_nbytes(v[1]) for v in model if v is not None)


def test_skip_cache_get_clears():
    c = EPSkipCache(3)
    t = torch.randn(4, 2)
    assert not c.contains(1) and c.tensors_size() == 0
    c.put(1, t)
    assert c.contains(1) and c.tensors_size() == _nbytes(t)
    assert c.get(1) is t
    assert not c.contains(1) and c.get(1) is None
    c.put(2, t)
    c.clear()
    assert not c.contains(2)
    assert EPSkipCache(0).tensors_size() == 0
