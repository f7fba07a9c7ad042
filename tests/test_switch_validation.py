"""Constructor checks of the holder classes: they come before any device work, so they run on CPU.
The messages are the reference's (src/ramp/nn/switch_linear.py:121-150, glm4_moe_adapter.py:124-135)."""

import numpy as np
import pytest
import torch

from keep_b200._lib import KeepVQError
from keep_b200.switch import QuantizedVQSwitchGLU, QuantizedVQSwitchLinear


def arrays(experts=3, out=8, inp=64, group=32):
    codes = torch.from_numpy(np.zeros((experts, out, inp // 8), dtype=np.uint16))
    scales = torch.ones((experts, out, inp // group), dtype=torch.float16)
    return dict(input_dims=inp, output_dims=out, num_experts=experts, codes=codes, scales=scales, group_size=group, code_bits=16)


@pytest.mark.parametrize("change,message", [
    (dict(output_dims=0), "must be positive"), (dict(input_dims=60), "divisible by 8"), (dict(group_size=24), "divisible by group_size"),
    (dict(code_bits=12), "code_bits must be 8 or 16"), (dict(gather_codebook_duplication=3), "must be 1, 4, or 8"),
    (dict(route_strategy="sorted"), "route_strategy must be"), (dict(num_experts=4), "codes must have shape"),
    (dict(bias=torch.zeros((3, 7))), "bias must have shape")])
def test_linear_rejects_bad_metadata(change, message):
    with pytest.raises(ValueError, match=message):
        QuantizedVQSwitchLinear(**{**arrays(), **change})


def test_linear_refuses_conversion_sidecars_and_cpu_tensors():
    with pytest.raises(NotImplementedError, match="rotation_matrix"):
        QuantizedVQSwitchLinear(**arrays(), rotation_matrix=torch.eye(64))
    with pytest.raises(TypeError, match="unexpected keyword"):
        QuantizedVQSwitchLinear(**arrays(), shuffle=True)
    with pytest.raises(KeepVQError, match="no CPU path"):  # valid metadata, but the tensors are on the host
        QuantizedVQSwitchLinear(**arrays())


class Shape:  # the GLU constructor only looks at dimensions and expert counts
    def __init__(self, inp, out, experts=4):
        self.input_dims, self.output_dims, self.num_experts = inp, out, experts


def test_glu_rejects_mismatched_projections():
    ok = dict(gate_proj=Shape(64, 32), up_proj=Shape(64, 32), down_proj=Shape(32, 64))
    QuantizedVQSwitchGLU(**ok)
    for change, message in ((dict(up_proj=Shape(48, 32)), "input dimensions must match"), (dict(up_proj=Shape(64, 16)), "output dimensions must match"),
                            (dict(down_proj=Shape(16, 64)), "down_proj input dimension"), (dict(down_proj=Shape(32, 48)), "down_proj output dimension"),
                            (dict(down_proj=Shape(32, 64, 5)), "same expert count"), (dict(prefill_engine="cuda"), "prefill_engine must be")):
        with pytest.raises(ValueError, match=message):
            QuantizedVQSwitchGLU(**{**ok, **change})
