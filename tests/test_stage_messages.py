"""Messages between the orchestrator and stage processes carry host data only."""
import pytest
import torch

from vllm_omni_b200.entrypoints.stage_utils import to_host
from vllm_omni_b200.outputs import CompletionOutput, RequestOutput


def _message(dev):
    c = CompletionOutput(index=0, text="", token_ids=[1], finish_reason=None, stop_reason=None)
    c.multimodal_output = {"codes": torch.ones(4, 2, dtype=torch.long, device=dev), "n": 3}
    ro = RequestOutput(request_id="r", prompt=None, prompt_token_ids=[1], outputs=[c], finished=True, metrics={},
                       multimodal_output=c.multimodal_output)
    return {"engine_outputs": [ro], "extra": (torch.zeros(1, device=dev), "x"), "loop": None}


def test_to_host_walks_containers_and_output_objects():
    m = _message("cpu")
    m["loop"] = m                                             # cycles do not recurse forever
    out = to_host(m)
    assert out is m and out["engine_outputs"][0].outputs[0].multimodal_output["n"] == 3
    assert isinstance(out["extra"], tuple) and out["extra"][1] == "x"


@pytest.mark.gpu
def test_to_host_moves_cuda_tensors():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    out = to_host(_message("cuda"))
    mm = out["engine_outputs"][0].outputs[0].multimodal_output
    assert not mm["codes"].is_cuda and not out["extra"][0].is_cuda and not out["engine_outputs"][0].multimodal_output["codes"].is_cuda
