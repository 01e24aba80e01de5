"""Host-side refusals around the kernels: wrong device, and the device status word.

None of these needs a GPU: the device check is a pure function over
``torch.device`` values, and the status paths are driven by writing the status
word from the host, as a kernel whose bounded wait ran out would have.
"""

import pytest
import torch

from aotolith_b200 import ops
from aotolith_b200.errors import DeviceError
from aotolith_b200.models.session import DecodeSession
from aotolith_b200.peer import PeerSum


def test_operands_must_sit_on_the_current_device():
    cuda0, cuda1 = torch.device("cuda", 0), torch.device("cuda", 1)
    ops.check_operand_devices([cuda0, cuda0, torch.device("cuda")], 0)   # plain "cuda" = current
    ops.check_operand_devices([], 3)
    with pytest.raises(DeviceError, match="different GPUs"):
        ops.check_operand_devices([cuda0, cuda1], 0)
    with pytest.raises(DeviceError, match="current CUDA device is cuda:0"):
        ops.check_operand_devices([cuda1, cuda1], 0)
    with pytest.raises(DeviceError, match="CUDA tensors"):
        ops.check_operand_devices([torch.device("cpu")], 0)


def test_cpu_tensors_are_refused_by_the_wrappers():
    x = torch.zeros(1, 64, dtype=torch.bfloat16)
    with pytest.raises(DeviceError):
        ops.rms_norm(x, torch.ones(64, dtype=torch.bfloat16), 1e-6)


def test_session_status_word_becomes_a_device_error():
    """A step kernel that gave up leaves 1 + the stage index in ``status``."""

    session = DecodeSession.__new__(DecodeSession)
    session.status = torch.tensor([8], dtype=torch.int32)
    session.scratch = torch.ones(64, dtype=torch.uint8)
    session.arena = torch.ones(64, dtype=torch.uint8)
    with pytest.raises(DeviceError, match="stage 7"):
        session._check_status()
    assert int(session.status) == 0 and not session.scratch.any() and not session.arena.any()
    session._check_status()  # a clear word is not an error


def test_peer_sum_status_word_becomes_a_device_error():
    exchange = PeerSum.__new__(PeerSum)
    exchange.status = torch.tensor([1], dtype=torch.int32)
    with pytest.raises(DeviceError, match="peer-exchange poll ran out"):
        exchange.check()
    assert int(exchange.status) == 0
    exchange.check()
