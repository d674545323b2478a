"""A tour of the request-level features on the tiny random-weight model (runs on a CPU in seconds):

    python examples/features_tour.py

structured output (regex / JSON schema / choice), log-probabilities of prompt and output, beam search,
embeddings, n-gram speculative decoding, and prefix caching. The same calls work on a checkpoint directory
with ``tensor_parallel_size=8`` on GPUs.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tokenweave_b200 import LLM, BeamSearchParams, SamplingParams  # noqa: E402


def main():
    llm = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=256, seed=0,
              enable_prefix_caching=True, speculative_config={"method": "ngram", "num_speculative_tokens": 3})

    date = llm.generate(["Today is "], SamplingParams(temperature=1.0, seed=1, max_tokens=16,
                                                     guided_regex=r"20\d{2}-(0[1-9]|1[0-2])-(0[1-9]|[12]\d)"))[0]
    print("regex      :", date.outputs[0].text)

    schema = {"type": "object", "properties": {"name": {"type": "string", "maxLength": 6}, "ok": {"type": "boolean"}},
              "required": ["name", "ok"]}
    doc = llm.generate(["JSON: "], SamplingParams(temperature=1.0, seed=2, max_tokens=64, guided_json=schema))[0]
    print("json schema:", json.loads(doc.outputs[0].text))

    grammar = '''
        root ::= expr
        expr ::= term (("+" | "-") term)*
        term ::= [1-9] [0-9]? | "(" expr ")"
    '''
    calc = llm.generate(["calc: "], SamplingParams(temperature=1.0, seed=4, max_tokens=40, guided_grammar=grammar))[0]
    print("grammar    :", calc.outputs[0].text)

    pick = llm.generate(["Colour? "], SamplingParams(temperature=1.0, seed=3, max_tokens=8,
                                                    guided_choice=["red", "green", "blue"]))[0]
    print("choice     :", pick.outputs[0].text)

    lp = llm.generate(["abc"], SamplingParams(temperature=0, max_tokens=2, logprobs=2, prompt_logprobs=1))[0]
    print("logprobs   :", [round(max(d.values()), 3) for d in lp.outputs[0].logprobs],
          "| prompt:", [None if d is None else round(max(d.values()), 3) for d in lp.prompt_logprobs])

    beams = llm.beam_search(["Once"], BeamSearchParams(beam_width=3, max_tokens=4))[0]
    print("beam search:", [round(s.cum_logprob, 3) for s in beams.sequences])

    a, b = llm.embed(["hello world", "hello there"])
    print("embeddings :", tuple(a.data.shape), "cosine", round(float((a.data * b.data).sum()), 4))

    rep = llm.generate(["abcabcabcabc"], SamplingParams(temperature=0, max_tokens=12, ignore_eos=True))[0]
    sched = llm.llm_engine.core.scheduler
    print("spec decode:", len(rep.outputs[0].token_ids), "tokens,", sched.num_accepted_tokens, "of",
          sched.num_draft_tokens, "drafts confirmed")
    llm.shutdown()

    # 8-bit weights and activations (on a GPU: the tcgen05 kind::i8 GEMM; here the reference arithmetic)
    q = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=256, seed=3,
            quantization="int8")
    out = q.generate(["abc"], SamplingParams(temperature=0, max_tokens=4))[0]
    print("int8 model :", out.outputs[0].token_ids)
    q.shutdown()


if __name__ == "__main__":
    main()
