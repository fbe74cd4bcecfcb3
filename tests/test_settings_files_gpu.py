"""Files beside config.json that change how a model folder is served: generation_config.json."""
import json

import numpy as np
import pytest

from helpers import TINY, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


def test_generation_config_file_names_the_end_tokens(tmp_path):
    """generation_config.json beside config.json replaces the model configuration's end-of-sequence
    ids, as in the reference (rust/engine/src/runner/model/qwen2/engine.rs:403-407); a request's own
    ids still come first."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    cfg, opt = TINY["A"]
    folder = make_model_folder(str(tmp_path / "model"), cfg, opt["seed"], "float32")
    prompt = random_tokens(np.random.default_rng(8), 7, cfg["vocab_size"])
    llm = LLM(folder, "f32", page_size=opt["page_size"], kv_tokens=128, max_requests=2)
    assert llm.model_eos == [cfg["eos_token_id"]]
    free = llm.generate([prompt], SamplingConfig(max_new_tokens=6, ignore_eos=True))[0].tokens
    del llm
    other = next(t for t in range(cfg["vocab_size"]) if t not in free)     # a second id that never comes
    with open(f"{folder}/generation_config.json", "w") as fh:
        json.dump({"eos_token_id": [free[2], other], "temperature": 0.7, "do_sample": True}, fh)
    llm = LLM(folder, "f32", page_size=opt["page_size"], kv_tokens=128, max_requests=2)
    assert llm.model_eos == [free[2], other]
    res = llm.generate([prompt], SamplingConfig(max_new_tokens=6))[0]
    assert res.tokens == free[: free.index(free[2]) + 1] and res.finish_reason == "eos"
    own = llm.generate([prompt], SamplingConfig(max_new_tokens=6, eos_token_id=free[1]))[0]
    assert own.tokens == free[: free.index(free[1]) + 1] and own.finish_reason == "eos"
