"""Argument checks of Engine.forward that run before any pointer reaches the library (no GPU needed): a host
tensor, a short buffer or a wrong dtype must raise ValueError instead of becoming a bad device address."""
import pytest
import torch

from chessrl_b200 import _lib as L
from chessrl_b200.engine import check_forward_inputs, check_rows

DEV = torch.device("cuda", 0)      # the engine's device in these checks; no CUDA call is made
CPU = torch.device("cpu")


class FakeCuda:
    """Stands for a tensor on cuda:0 without touching a GPU: only the attributes the checks read."""

    def __init__(self, shape, dtype, index=0):
        self.shape, self.dtype, self.device = torch.Size(shape), dtype, torch.device("cuda", index)

    def dim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n


def test_check_rows_rejects_device_dtype_and_length():
    good = FakeCuda((4, 233), torch.uint8)
    check_rows("legal_mask", good, DEV, 4, (torch.uint8, torch.float32))
    with pytest.raises(ValueError, match="must live on"):
        check_rows("legal_mask", torch.zeros(4, 233, dtype=torch.uint8), DEV, 4, (torch.uint8,))
    with pytest.raises(ValueError, match="must live on"):
        check_rows("legal_mask", FakeCuda((4, 233), torch.uint8, index=1), DEV, 4, (torch.uint8,))
    with pytest.raises(ValueError, match="rows"):
        check_rows("legal_mask", FakeCuda((3, 233), torch.uint8), DEV, 4, (torch.uint8,))
    with pytest.raises(ValueError, match="dtype"):
        check_rows("legal_mask", FakeCuda((4, 233), torch.int64), DEV, 4, (torch.uint8, torch.float32))


def test_forward_input_rules_host_side():
    b = 5
    planes = torch.zeros(b, 8, 8, 112, dtype=torch.float16)
    bits = torch.zeros(b, 233, dtype=torch.uint8)
    check_forward_inputs(planes, CPU, b, 1858, bits, None, torch.zeros(b, dtype=torch.uint8), torch.zeros(b), True)
    with pytest.raises(ValueError, match="planes must live on"):
        check_forward_inputs(planes, DEV, b, 1858)
    with pytest.raises(ValueError, match="rows"):
        check_forward_inputs(planes, CPU, b, 1858, bits[:3])
    with pytest.raises(ValueError, match="needs 233"):
        check_forward_inputs(planes, CPU, b, 1858, bits[:, :200])
    with pytest.raises(ValueError, match="needs 1858"):
        check_forward_inputs(planes, CPU, b, 1858, torch.zeros(b, 233))          # float32 rows must span the moves
    with pytest.raises(ValueError, match="dtype"):
        check_forward_inputs(planes, CPU, b, 1858, bits.to(torch.int32))
    with pytest.raises(ValueError, match="mask_mode"):
        check_forward_inputs(planes, CPU, b, 1858, bits, L.MASK_ADDITIVE)
    with pytest.raises(ValueError, match="black_rows"):
        check_forward_inputs(planes, CPU, b, 1858, black_rows=torch.zeros(b - 1, dtype=torch.uint8), rl_vocab=True)
    with pytest.raises(ValueError, match="uniforms"):
        check_forward_inputs(planes, CPU, b, 1858, uniforms=torch.zeros(b + 1))


def test_device_tensors_are_required_for_the_device_entry():
    """host=False: a CPU mask or CPU black_rows next to device planes is refused."""
    b = 4
    planes = FakeCuda((b, 8, 8, 112), torch.float16)
    with pytest.raises(ValueError, match="legal_mask must live on"):
        check_forward_inputs(planes, DEV, b, 1858, torch.zeros(b, 233, dtype=torch.uint8))
    with pytest.raises(ValueError, match="black_rows must live on"):
        check_forward_inputs(planes, DEV, b, 1858, FakeCuda((b, 233), torch.uint8), None,
                             torch.zeros(b, dtype=torch.uint8), None, True)
    check_forward_inputs(planes, DEV, b, 1858, FakeCuda((b, 233), torch.uint8), None, FakeCuda((b,), torch.uint8),
                         FakeCuda((b,), torch.float32), True)
