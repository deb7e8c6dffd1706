"""Agentic training support: tools and environments, multi-turn rollouts (sampler- or API-driven), context chunking
and condensing, a confidence-routed sampler, answer-overlap rewards and trajectory quality filters
(reference package ``twinkle_agentic``)."""
from .context import (Chunk, Chunker, Chunks, Condenser, ExtractCondensed, KeywordCondenser, ModelCondenser, MultiTurnCondenseRollout,
                      NativeChunker)
from .openenv import EnvPoolAdapter, OpenEnv, ShardedEnvPool, normalize_result, observation_text
from .pii import PIIPresidioFilter, PIIRewriter, Strategy
from .preprocess import (ChrMinScorer, CodeDetector, ComplexLogicDetector, FixUnicodeFilter, IntentClassifier, IntentDetector, LLMBackend,
                         MathDetector, MessageNormalizer, ModelFilter, OpenAIBackend, ParaphraseScorer, PassNScorer, QualityPreprocessor,
                         ReasoningDetector, RemoveRepeatSentencesFilter, RoundContext, RoundScoreFilter, SamplerBackend, ScoreResult,
                         SIFDScorer, SpecialCharsFilter, TokenNumFilter, ToolCallDetector, UserDissatisfactionDetector,
                         chr_min_distinct, count_tokens, ifd_family, special_char_ratio)
from .quality import (CoTReward, DeadLoopFilter, DedupFilter, F1Reward, HardFilter, MessageSanityFilter, PIIFilter, RefuseFilter,
                      RouterSampler, ScoreFilter, TokenSoupFilter, ToolExploreReward, f1_score, normalize_messages)
from .rollout import (APIMultiTurnRollout, ChatAPI, MultiTurnRollout, OpenAIChatAPI, Rollout, extend_with_bridge, parse_tool_calls,
                      strip_tool_calls)
from .tools import Env, EnvPool, EnvTool, FunctionTool, StepResult, Tool, ToolManager

__all__ = [n for n in dir() if not n.startswith('_')]
