"""The step arena on the CPU: offsets bumped region by region, a layer's region reused two
layers later, the same addresses step after step, growth by one kept block, and tensors too
large for a region left to the allocator."""

import torch

from kv_cache_optimization_for_llm_b200.engine.arena import StepArena


def _addresses(a, layers=4):
    out = []
    a.begin_step()
    out.append(a.new((10, 16), torch.float32).data_ptr())          # the residual: lives for the step
    for _ in range(layers):
        a.begin_layer()
        out.append((a.new((10, 48), torch.bfloat16).data_ptr(), a.new((10, 16), torch.bfloat16).data_ptr()))
    a.end_layers()
    out.append(a.new((2, 100), torch.float32).data_ptr())          # logits
    return out


def test_regions_alternate_and_addresses_repeat():
    a = StepArena("cpu", step_bytes=4096, layer_bytes=4096)
    first = _addresses(a)
    # layers 0 and 2 share a region, layers 1 and 3 the other; neighbours never share
    assert first[1] == first[3] and first[2] == first[4] and first[1] != first[2]
    # what lives for the step lies in a region of its own
    assert first[0] not in (first[1][0], first[2][0]) and first[5] != first[0]
    # a step of the same shape finds every tensor where the step before had it
    assert _addresses(a) == first
    assert a.blocks_grown() == 0 and a.bypassed == 0
    # tensors are aligned and do not overlap
    a.begin_step()
    x, y = a.new((3, 5), torch.bfloat16), a.new((7,), torch.int32)
    assert x.data_ptr() % 256 == 0 and y.data_ptr() % 256 == 0 and y.data_ptr() >= x.data_ptr() + 30
    x.fill_(1.0); y.fill_(7)
    assert float(x.sum()) == 15.0 and int(y.sum()) == 49


def test_a_region_that_is_too_small_grows_once_and_keeps_the_block():
    a = StepArena("cpu", step_bytes=1024, layer_bytes=1024)
    a.begin_step()
    a.begin_layer()
    t1 = a.new((200,), torch.float32)      # 800 bytes
    t2 = a.new((200,), torch.float32)      # does not fit behind it: a second block
    assert a.blocks_grown() == 1 and t1.data_ptr() != t2.data_ptr()
    held = a.bytes_held()
    a.begin_step()
    a.begin_layer()                         # the first layer's region again, with its two blocks
    assert (a.new((200,), torch.float32).data_ptr(), a.new((200,), torch.float32).data_ptr()) == (t1.data_ptr(), t2.data_ptr())
    assert a.blocks_grown() == 1 and a.bytes_held() == held
    # larger than a whole region: from the allocator, the arena untouched
    big = a.new((1000,), torch.float32)
    assert a.bypassed == 1 and big.numel() == 1000 and a.bytes_held() == held
    # nothing at all is a tensor too
    assert a.new((0, 5), torch.float32).shape == (0, 5)


def test_a_step_of_the_same_shape_gets_the_same_tensor_objects():
    """The arena keeps the tensors it has handed out, by place, type and shape: asking again costs a
    dictionary lookup, and another shape or type at the same place gets a tensor of its own."""
    a = StepArena("cpu", step_bytes=4096, layer_bytes=4096)

    def step(rows, dtype=torch.bfloat16):
        a.begin_step()
        resid = a.new((rows, 16), torch.float32)
        a.begin_layer()
        return resid, a.new((rows, 48), dtype), a.new([rows, 16], dtype)
    first = step(10)
    again = step(10)
    assert all(x is y for x, y in zip(first, again))
    other = step(6)
    assert other[0] is not first[0] and other[0].shape == (6, 16) and other[0].data_ptr() == first[0].data_ptr()
    typed = step(10, torch.float32)
    assert typed[1] is not first[1] and typed[1].dtype == torch.float32 and typed[1].data_ptr() == first[1].data_ptr()
    assert all(x is y for x, y in zip(step(10), first))     # and the first shape's tensors are still there
