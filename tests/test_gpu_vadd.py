"""Vector add on the GPU: bit-exact against x + y (the oracle)."""

import gc
import weakref

import numpy as np
import pytest
import torch

import oracle
import swage_b200 as sw
import swage_b200.language as sl

pytestmark = pytest.mark.gpu


@sw.jit
def add_kernel(x_ptr, y_ptr, output_ptr, n, BLOCK: sl.constexpr):  # noqa: D103
    pid = sl.program_id(0)
    offsets = pid * BLOCK + sl.arange(0, BLOCK)
    mask = offsets < n
    x = sl.load(x_ptr + offsets, mask=mask, other=0.0)
    y = sl.load(y_ptr + offsets, mask=mask, other=0.0)
    sl.store(output_ptr + offsets, x + y, mask=mask)


def launch(x, y, output, n, block=128):
    add_kernel.launch(
        arguments={"x_ptr": x, "y_ptr": y, "output_ptr": output, "n": n},
        constexprs={"BLOCK": block},
        grid=((n + block - 1) // block,),
    )


def same_bits(a, b):
    return torch.equal(a.view(torch.int32), b.view(torch.int32))


@pytest.mark.parametrize("block", [128, 1024])
@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 127, 128, 129, 1025, 4097,
                               (1 << 20) + 3, 4 * 1024 * 256 * 3 + 1])
def test_matches_the_oracle_bit_for_bit(n, block):
    x = torch.randn(n, device="cuda")
    y = torch.randn(n, device="cuda")
    output = torch.full((n + 5,), float("nan"), device="cuda")
    launch(x, y, output, n, block)
    torch.cuda.synchronize()
    expected = oracle.vadd_f32(x.cpu().numpy(), y.cpu().numpy(), n, block)
    assert np.array_equal(output[:n].cpu().numpy().view(np.uint32),
                          expected.view(np.uint32))
    assert torch.isnan(output[n:]).all(), "wrote past n"


@pytest.mark.parametrize("shifts", [(1, 1, 1), (1, 2, 3), (0, 3, 0),
                                    (2, 2, 0), (3, 3, 3)])
def test_four_byte_aligned_views(shifts):
    n = 100_003
    base = [torch.randn(n + 8, device="cuda") for _ in range(3)]
    x, y = base[0][shifts[0]:shifts[0] + n], base[1][shifts[1]:shifts[1] + n]
    base[2].fill_(float("nan"))
    output = base[2][shifts[2]:shifts[2] + n]
    launch(x, y, output, n)
    torch.cuda.synchronize()
    assert same_bits(output, x + y)
    assert torch.isnan(base[2][:shifts[2]]).all()
    assert torch.isnan(base[2][shifts[2] + n:]).all()


def test_n_smaller_than_the_tensors():
    x = torch.randn(1000, device="cuda")
    y = torch.randn(1000, device="cuda")
    output = torch.zeros(1000, device="cuda")
    launch(x, y, output, 600)
    torch.cuda.synchronize()
    assert same_bits(output[:600], (x + y)[:600])
    assert (output[600:] == 0).all()


def test_special_values_are_bit_exact():
    specials = torch.tensor(
        [0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1e-45, -1e-45,
         3.4028235e38, -3.4028235e38, 1.0], device="cuda")
    x = specials.repeat_interleave(10)
    y = specials.repeat(10)
    output = torch.empty_like(x)
    launch(x, y, output, x.numel())
    torch.cuda.synchronize()
    expected = x + y
    both_nan = torch.isnan(output) & torch.isnan(expected)
    assert torch.all(both_nan | (output.view(torch.int32)
                                 == expected.view(torch.int32)))


def test_uses_the_current_stream_without_synchronising():
    x = torch.randn(129, device="cuda")
    y = torch.randn(129, device="cuda")
    output = torch.empty_like(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        launch(x, y, output, 129)
    stream.synchronize()
    assert same_bits(output, x + y)


def test_repeated_launches_release_their_arguments():
    def launch_local():
        x = torch.randn(129, device="cuda")
        y = torch.randn(129, device="cuda")
        output = torch.empty_like(x)
        references = (weakref.ref(x), weakref.ref(y), weakref.ref(output))
        launch(x, y, output, 129)
        launch(x, y, output, 129)
        torch.cuda.current_stream().synchronize()
        return references

    references = launch_local()
    gc.collect()
    assert all(reference() is None for reference in references)


def test_rejects_invalid_runtime_inputs():
    x = torch.empty(4, device="cuda")
    output = torch.empty_like(x)
    arguments = {"x_ptr": x, "y_ptr": x, "output_ptr": output, "n": 4}
    with pytest.raises(TypeError, match="must be a CUDA tensor"):
        add_kernel.launch(arguments={**arguments, "y_ptr": torch.empty(4)},
                          constexprs={"BLOCK": 128}, grid=(1,))
    with pytest.raises(ValueError, match="exceeds tensor length"):
        add_kernel.launch(arguments={**arguments, "n": 5},
                          constexprs={"BLOCK": 128}, grid=(1,))
    with pytest.raises(ValueError, match="grid must equal"):
        add_kernel.launch(arguments=arguments, constexprs={"BLOCK": 128},
                          grid=(2,))
    limit = torch.cuda.get_device_properties(
        torch.cuda.current_device()).max_threads_per_block
    with pytest.raises(ValueError, match="exceeds device limit"):
        add_kernel.launch(arguments=arguments,
                          constexprs={"BLOCK": limit + 1}, grid=(1,))


def test_full_size_configuration():
    """n = 2**28 - 37, BLOCK 128 and 1024: bit-exact against x + y."""
    n = (1 << 28) - 37
    x = torch.randn(n, device="cuda")
    y = torch.randn(n, device="cuda")
    expected = x + y
    for block in (128, 1024):
        output = torch.empty(n, device="cuda")
        launch(x, y, output, n, block)
        torch.cuda.synchronize()
        assert same_bits(output, expected)
        del output
