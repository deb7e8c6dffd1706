"""Row → trajectory converters for common public datasets.

Parity: reference ``src/twinkle/preprocessor/*.py`` (``Preprocessor`` batched row→row, ``DataFilter``;
Alpaca, SelfCognition, GSM8K, CompetitionMath, Countdown, EmojiDPO, CLEVR, OlympiadBench)."""
from __future__ import annotations

import re
from typing import Any, Dict, List, Optional


class Preprocessor:
    """``__call__`` takes and returns a list of rows; override ``preprocess(row)`` for the 1:1 case (return None to drop)."""

    def __call__(self, rows: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
        out = []
        for r in rows:
            y = self.preprocess(r)
            if y is None:
                continue
            out.extend(y if isinstance(y, list) else [y])
        return out

    def preprocess(self, row: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        return row


class DataFilter(Preprocessor):

    def keep(self, row: Dict[str, Any]) -> bool:
        return True

    def preprocess(self, row):
        return row if self.keep(row) else None


def _traj(user: str, assistant: Optional[str] = None, system: Optional[str] = None, **extra) -> Dict[str, Any]:
    msgs = []
    if system:
        msgs.append({'role': 'system', 'content': system})
    msgs.append({'role': 'user', 'content': user})
    if assistant is not None:
        msgs.append({'role': 'assistant', 'content': assistant})
    return {'messages': msgs, **extra}


class AlpacaProcessor(Preprocessor):

    def preprocess(self, row):
        q = row.get('instruction', '')
        if row.get('input'):
            q = f"{q}\n{row['input']}"
        return _traj(q, row.get('output', ''))


class SelfCognitionProcessor(Preprocessor):

    def __init__(self, model_name: str = 'twinkle', model_author: str = 'modelscope'):
        self.name, self.author = model_name, model_author

    def preprocess(self, row):
        rep = lambda s: s.replace('{{NAME}}', self.name).replace('{{AUTHOR}}', self.author)
        return _traj(rep(row.get('query', '')), rep(row.get('response', '')))


class GSM8KProcessor(Preprocessor):
    SYSTEM = 'Solve the problem step by step and finish with "#### <number>".'

    def preprocess(self, row):
        return _traj(row['question'], row.get('answer'), self.SYSTEM, user_data={'ground_truth': str(row.get('answer', '')).split('####')[-1].strip()})


class GSM8KPromptProcessor(GSM8KProcessor):
    """Prompt only (RL): the answer moves to ``user_data``."""

    def preprocess(self, row):
        t = super().preprocess(row)
        t['messages'] = [m for m in t['messages'] if m['role'] != 'assistant']
        return t


class CompetitionMathProcessor(Preprocessor):

    def preprocess(self, row):
        return _traj(row.get('problem', ''), row.get('solution'), 'Put the final answer in \\\\boxed{}.', user_data={'ground_truth': row.get('solution', '')})


class CompetitionMathGRPOProcessor(Preprocessor):
    """Prompt-only rows for RL on competition math: the policy is told to answer with the boxed result alone; the worked
    solution travels in ``user_data`` (``solution`` and, extracted from its last ``\\boxed{}``, ``ground_truth``)."""

    def preprocess(self, row):
        from ..reward import extract_boxed
        sol = row.get('solution', '')
        return _traj(row.get('problem', ''), None, 'You are a helpful math assistant. Respond with only the final answer in the form '
                     '\\boxed{...} and nothing else.', user_data={'solution': sol, 'ground_truth': extract_boxed(sol) or sol})


class CountdownProcessor(Preprocessor):

    def preprocess(self, row):
        nums, target = row['nums'], row['target']
        q = f'Using the numbers {nums}, create an equation that equals {target}. Use each number once. Answer inside <answer></answer>.'
        return _traj(q, None, user_data={'ground_truth': {'nums': list(nums), 'target': target}})


class EmojiDPOProcessor(Preprocessor):
    """One preference row → two interleaved trajectories (chosen first)."""

    def preprocess(self, row):
        return [_traj(row['prompt'], row['chosen']), _traj(row['prompt'], row['rejected'])]


class CLEVRProcessor(Preprocessor):

    def preprocess(self, row):
        """Visual question answering rows (``problem`` / ``question``, ``solution`` possibly wrapped in ``<answer>`` tags, ``image``):
        the image goes to ``images`` (the vision-language template places it before the question), the answer also to
        ``user_data`` for the multimodal accuracy reward."""
        sol = row.get('solution')
        t = _traj(row.get('problem', row.get('question', '')), sol)
        if row.get('image') is not None:
            t['images'] = [row['image']]
        if sol is not None:
            m = re.search(r'<answer>\s*(.*?)\s*</answer>', str(sol), re.S)
            t['user_data'] = {'solution': sol, 'ground_truth': m.group(1) if m else str(sol)}
        return t


class OlympiadBenchProcessor(Preprocessor):

    def preprocess(self, row):
        ans = row.get('final_answer')
        ans = ans[0] if isinstance(ans, list) and ans else ans
        return _traj(row.get('question', ''), None, 'Reason step by step; final answer in \\\\boxed{}.', user_data={'ground_truth': ans})


class MaxLengthFilter(DataFilter):

    def __init__(self, max_chars: int = 32768):
        self.max_chars = max_chars

    def keep(self, row):
        return sum(len(str(m.get('content', ''))) for m in row.get('messages', [])) <= self.max_chars


preprocessor_mapping = {c.__name__: c for c in (AlpacaProcessor, SelfCognitionProcessor, GSM8KProcessor, GSM8KPromptProcessor, CompetitionMathGRPOProcessor,
                                                CompetitionMathProcessor, CountdownProcessor, EmojiDPOProcessor, CLEVRProcessor,
                                                OlympiadBenchProcessor, MaxLengthFilter)}
