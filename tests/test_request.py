"""Request state and sampling parameters (shrike tests/test_request.py:16-78)."""

import pytest

from shrike_b200 import SamplingParams
from shrike_b200.engine.request import Request, Status


def test_defaults_and_bounds():
    params = SamplingParams()
    assert (params.max_new_tokens, params.temperature, params.top_p, params.ignore_eos) == (128, 0.0, 1.0, False)
    for bad in (dict(max_new_tokens=0), dict(temperature=-0.1), dict(top_p=0.0), dict(top_p=1.5)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
    SamplingParams(top_p=1.0, temperature=0.0, max_new_tokens=1)


def test_request_counters():
    a = Request(token_ids=[1, 2, 3], sampling=SamplingParams())
    b = Request(token_ids=[4], sampling=SamplingParams())
    assert b.req_id > a.req_id
    assert a.status is Status.WAITING and a.num_prompt_tokens == 3 and not a.prefill_done
    a.num_computed_tokens = 3
    a.token_ids.append(9)
    assert a.prefill_done and a.num_generated == 1 and a.num_tokens == 4 and a.num_prompt_tokens == 3
    assert a.block_table == []
