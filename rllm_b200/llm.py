"""The Python entry point, shaped like the reference's blocking engine
(crates/rllm-engine/src/sync_engine.rs:10-64: ``add_request``, ``step``,
``has_work`` and a ``generate`` that steps until every request has finished).

    from rllm_b200 import LLM, SamplingParams
    llm = LLM("path/to/model", dtype="bf16")
    outs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=32))
    outs[0].outputs[0].token_ids

Prompts are token ids: tokenisation is outside this engine.  Keyword options
carry the names of ``rllm serve`` (crates/rllm-server/src/cli.rs:27-49).
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence, Union

from .config.engine_args import EngineArgs
from .engine.engine_core import CompletionOutput, EngineCore, RequestOutput, Usage
from .engine.loading import load_model
from .sampling import SamplingParams


class LLM:
    def __init__(self, model: str, dtype: str = "auto", max_model_len: Optional[int] = None,
                 max_num_seqs: int = 256, max_num_batched_tokens: int = 4096,
                 gpu_memory_utilization: float = 0.9, enable_prefix_caching: bool = True,
                 block_size: int = 16, num_gpu_blocks: Optional[int] = None,
                 long_prefill_token_threshold: int = 2048, enable_chunked_prefill: bool = True,
                 enable_cuda_graphs: bool = True, random_weights: bool = False, seed: int = 0,
                 device: Optional[str] = None, draw_on_device: bool = False, step_row_multiple: int = 128,
                 scheduling_policy: str = "fcfs"):
        self.args = EngineArgs(dtype=dtype, max_model_len=max_model_len, max_num_seqs=max_num_seqs,
                               max_num_batched_tokens=max_num_batched_tokens,
                               gpu_memory_utilization=gpu_memory_utilization,
                               enable_prefix_caching=enable_prefix_caching, block_size=block_size,
                               num_gpu_blocks=num_gpu_blocks,
                               long_prefill_token_threshold=long_prefill_token_threshold,
                               enable_chunked_prefill=enable_chunked_prefill,
                               enable_cuda_graphs=enable_cuda_graphs, seed=seed,
                               step_row_multiple=step_row_multiple, scheduling_policy=scheduling_policy)
        self.args.validate()
        self.config, self.model = load_model(model, dtype=dtype, device=device,
                                             random_weights=random_weights, seed=seed,
                                             draw_on_device=draw_on_device)
        self.engine = EngineCore(self.model, self.args)

    # -- the reference's three calls ------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None, priority: int = 0) -> Hashable:
        return self.engine.add_request(prompt_token_ids, sampling_params, request_id, priority)

    def step(self) -> List[RequestOutput]:
        return self.engine.step()

    def has_work(self) -> bool:
        return self.engine.has_work()

    def abort_request(self, request_id: Hashable) -> bool:
        return self.engine.abort_request(request_id)

    # -- blocking generation ---------------------------------------------------
    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 priorities: Optional[Sequence[int]] = None) -> List[RequestOutput]:
        """One RequestOutput per prompt, in the order of the prompts, each with all generated
        tokens: ``outputs[i]`` is sample i of the prompt (one sample unless ``n`` > 1).
        ``priorities``: one per prompt, for the priority policy."""
        n = len(prompt_token_ids)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or SamplingParams()] * n
        else:
            params = list(sampling_params)
            if len(params) != n:
                raise ValueError("one SamplingParams per prompt, or one for all")
        if priorities is not None and len(priorities) != n:
            raise ValueError("one priority per prompt")
        ids = [self.add_request(p, sp, priority=0 if priorities is None else int(priorities[i]))
               for i, (p, sp) in enumerate(zip(prompt_token_ids, params))]
        # per request: sample index -> [tokens, log-probabilities, finish reason]
        samples = {rid: {i: [[], [], None] for i in range(sp.n)} for rid, sp in zip(ids, params)}
        while self.has_work():
            for out in self.step():
                mine = samples.get(out.request_id)
                if mine is None:
                    continue
                for c in out.outputs:
                    got = mine[c.index]
                    got[0].extend(c.token_ids)
                    if c.logprobs is not None:
                        got[1].extend(c.logprobs)
                    if c.finish_reason is not None:
                        got[2] = c.finish_reason
        self.engine.runner.check_errors()          # the steps polled the kernels' error words; this waits for the last
        results = []
        for rid, prompt, sp in zip(ids, prompt_token_ids, params):
            # a sample without a reason was aborted from outside (``abort_request``) while this call was
            # stepping: what it had generated by then is returned, with the reference's reason for it
            # (crates/rllm-core/src/output.rs:37-42)
            outs = [CompletionOutput(i, toks, reason or "aborted", lps if sp.logprobs is not None else None)
                    for i, (toks, lps, reason) in sorted(samples[rid].items())]
            prompt = [int(t) for t in prompt]
            n_out = sum(len(o.token_ids) for o in outs)
            results.append(RequestOutput(rid, prompt, outs, True, Usage(len(prompt), n_out, len(prompt) + n_out)))
        return results
