"""Reinforcement learning: environments, advantage estimation, policies, storage, losses and the PPO / DQN / SAC trainers
(Source/Public/Oa/Ml/Rl/*.h of the reference)."""
from .environment import (OaCartPoleConfig, OaCartPoleEnvironment, OaLunarLander3dConfig, OaLunarLander3dEnvironment, OaRlEnvironment, OaRlEnvironmentSpec, OaRlEnvironmentTransition,
                          OaRlFieldSpec, OaRlSpaceKind)
from .fn_rl import (OaDqnLossConfig, OaDqnLossResult, OaGaeConfig, OaGaeResult, OaPpoLossConfig, OaPpoLossResult,
                    OaRlContinuousPolicyResult, OaRlPolicyResult, OaSacCriticLossResult, OaSacLossConfig)
from .storage import (OaRlReplayBatch, OaRlReplayBuffer, OaRlReplayConfig, OaRlReplayTransition, OaRlRolloutBatch, OaRlRolloutBuffer,
                      OaRlRolloutConfig, OaRlTransition)
from .trainers import (CopyModel, OaCategoricalActorCritic, OaCategoricalActorCriticConfig, OaDqnTrainer, OaDqnTrainerConfig,
                       OaDqnTrainerMetrics, OaItRlTraining, OaItRlTrainingConfig, OaPpoTrainer, OaPpoTrainerConfig, OaPpoTrainerMetrics,
                       OaRlActorCritic, OaRlActorCriticOutput, OaRlCollector, OaRlCollectorConfig, OaRlCollectorMetrics,
                       OaRlEvaluationConfig, OaRlEvaluationMetrics, OaRlTrainingPhase, OaSacTrainer, OaSacTrainerConfig,
                       OaSacTrainerMetrics)
from . import fn_rl as _fn


class OaFnRl:
    """Namespace of the RL matrix functions (Gae.h, Policy.h, Transform.h, Evaluation.h)."""
    Gae = staticmethod(_fn.Gae)
    GaeInto = staticmethod(_fn.GaeInto)
    NormalizeAdvantages = staticmethod(_fn.NormalizeAdvantages)
    SampleCategoricalPolicy = staticmethod(_fn.SampleCategoricalPolicy)
    EvaluateCategoricalPolicy = staticmethod(_fn.EvaluateCategoricalPolicy)
    SampleTanhNormalPolicy = staticmethod(_fn.SampleTanhNormalPolicy)
    EvaluateTanhNormalPolicy = staticmethod(_fn.EvaluateTanhNormalPolicy)
    NormalizeObservation = staticmethod(_fn.NormalizeObservation)
    ScaleAction = staticmethod(_fn.ScaleAction)
    ClipReward = staticmethod(_fn.ClipReward)
    SampleLogits = staticmethod(_fn.SampleLogits)

    @staticmethod
    def EvaluateCategorical(environment, model, config=None):
        from .trainers import EvaluateCategorical
        return EvaluateCategorical(environment, model, config)


class OaFnRlLoss:
    """The RL members of the OaFnLoss namespace (Rl/FnLoss.h)."""
    PpoClippedPolicy = staticmethod(_fn.PpoClippedPolicy)
    PpoClippedPolicyBwd = staticmethod(_fn.PpoClippedPolicyBwd)
    Ppo = staticmethod(_fn.Ppo)
    Dqn = staticmethod(_fn.Dqn)
    SacCritic = staticmethod(_fn.SacCritic)
    SacActor = staticmethod(_fn.SacActor)
