"""Rule-based scoring functions keyed by ``data_source`` (verl/utils/reward_score/__init__.py:19).

``default_compute_score(data_source, solution_str, ground_truth, extra_info)`` dispatches to the scorer of
the dataset family: GSM8K, MATH (+ DAPO variant), geometry3k, search-R1 exact match, code via a sandbox
service, and the two synthetic token rules used by the benchmark configs.
"""

from __future__ import annotations

from . import geo3k, gsm8k, math_dapo, math_reward, search_r1_like_qa_em, synthetic


def default_compute_score(data_source, solution_str, ground_truth, extra_info=None, sandbox_fusion_url=None,
                          concurrent_semaphore=None, memory_limit_mb=None, **kwargs):
    if data_source == "synthetic/even_fraction":
        res = synthetic.even_fraction(solution_str, ground_truth, extra_info)
    elif data_source == "synthetic/even_fraction_threshold":
        res = synthetic.even_fraction(solution_str, ground_truth, extra_info, threshold=0.5)
    elif data_source == "synthetic/contains_token":
        res = synthetic.contains_token(solution_str, ground_truth, extra_info)
    elif data_source == "openai/gsm8k":
        res = gsm8k.compute_score(solution_str, ground_truth)
    elif data_source in ("lighteval/MATH", "DigitalLearningGmbH/MATH-lighteval", "HuggingFaceH4/MATH-500"):
        res = math_reward.compute_score(solution_str, ground_truth)
    elif data_source in ("math_dapo", "math", "math_dapo_reasoning") or str(data_source).startswith("aime"):
        res = math_dapo.compute_score(solution_str, ground_truth)
    elif data_source in ("numina_aops_forum", "numina_synthetic_math", "numina_amc_aime", "numina_synthetic_amc",
                         "numina_cn_k12", "numina_olympiads"):
        res = math_reward.compute_score(solution_str, ground_truth)
    elif data_source in ("codecontests", "apps", "codeforces", "taco"):
        if sandbox_fusion_url:
            from . import sandbox_fusion

            res = sandbox_fusion.compute_score(sandbox_fusion_url, concurrent_semaphore, memory_limit_mb, solution_str,
                                               ground_truth, continuous=True)
        else:
            raise NotImplementedError("code data sources need reward_model.sandbox_fusion.url")
    elif data_source in ("prime_math",) or str(data_source).startswith("numina_prime"):
        from . import prime_math

        res = float(prime_math.compute_score(solution_str, ground_truth)[0])
    elif data_source in ("prime_code", "livecodebench"):
        from . import prime_code

        res = prime_code.compute_score(solution_str, ground_truth, continuous=True)[0]
    elif data_source in ("hiyouga/geometry3k",):
        res = geo3k.compute_score(solution_str, ground_truth)
    elif data_source in ("searchR1_nq", "searchR1_triviaqa", "searchR1_popqa", "searchR1_hotpotqa",
                         "searchR1_2wikimultihopqa", "searchR1_musique", "searchR1_bamboogle"):
        res = search_r1_like_qa_em.compute_score(solution_str, ground_truth)
    else:
        raise NotImplementedError(f"Reward function is not implemented for {data_source=}")
    if isinstance(res, dict):
        return res
    if isinstance(res, (int, float, bool)):
        return float(res)
    return float(res[0])


_default_compute_score = default_compute_score

__all__ = ["default_compute_score"]
