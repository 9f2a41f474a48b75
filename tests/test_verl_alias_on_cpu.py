"""``import verl...`` resolves to this framework's modules."""


def test_alias_imports_share_module_objects():
    import verl
    import verl_b200
    from verl import DataProto
    from verl.protocol import DataProto as DP2
    from verl.single_controller.base import Worker, register  # noqa: F401
    from verl.trainer.ppo import core_algos
    from verl.utils.reward_score import default_compute_score  # noqa: F401

    import verl_b200.trainer.ppo.core_algos as real

    assert DataProto is verl_b200.DataProto is DP2
    assert core_algos is real or core_algos.compute_grpo_outcome_advantage is real.compute_grpo_outcome_advantage
    import verl.utils.config as vc
    import verl_b200.utils.config as rc

    assert vc.compose is rc.compose and verl.__name__ == "verl"


def test_reference_module_paths_with_another_home_here():
    from verl.experimental.reward_loop.reward_manager.limited import RateLimitedRewardManager
    from verl.trainer.config.algorithm import AlgoConfig  # noqa: F401
    from verl.utils.kernel.linear_cross_entropy import lmhead_logprob_entropy  # noqa: F401
    from verl.workers.fsdp_workers import ActorRolloutRefWorker
    from verl.workers.reward_manager.naive import NaiveRewardManager

    import verl_b200.experimental.reward_loop.reward_manager as rl
    import verl_b200.workers.engine_workers as ew
    import verl_b200.workers.reward_manager as rm

    assert ActorRolloutRefWorker is ew.ActorRolloutRefWorker and NaiveRewardManager is rm.NaiveRewardManager
    assert RateLimitedRewardManager is rl.RateLimitedRewardManager
