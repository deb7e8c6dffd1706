"""Messages → tokens.

Parity: reference ``src/twinkle/template/base.py:28-859`` — pre-pipeline
(default system prompt, reasoning-content normalisation, standard message
shape), chat-template rendering with labels on assistant turns only
(round-by-round prefix tokenisation), post-pipeline (``max_length`` strategies
raise / left / right / split / delete, attention fields, **labels rolled left by
one** so that ``labels[t]`` is the target of ``logits[t]``),
``concat_input_feature`` for RL (prompt ⊕ sampled tokens with labels only on
the sampled part), ``decode``.

The tokenizer is a Hugging Face tokenizer when ``model_id`` points at one; a
self-contained byte-level ChatML tokenizer otherwise (used by tests and by
random-init benchmarks, where no tokenizer files exist).
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np

from ..data_format import InputFeature, Message, Trajectory

IGNORE = -100


class ByteChatTokenizer:
    """UTF-8 bytes + a few ChatML control tokens.  ids 0..255 are bytes."""
    SPECIAL = ['<|pad|>', '<|im_start|>', '<|im_end|>', '<|endoftext|>', '<tool_call>', '</tool_call>', '<think>', '</think>',
               '<|vision_start|>', '<|image_pad|>', '<|vision_end|>', '<|video_pad|>']

    def __init__(self, vocab_size: int = 1024):
        self.special = {t: 256 + i for i, t in enumerate(self.SPECIAL)}
        self.inv = {v: k for k, v in self.special.items()}
        self.vocab_size = max(vocab_size, 256 + len(self.SPECIAL))
        self.pad_token_id = self.special['<|pad|>']
        self.eos_token_id = self.special['<|im_end|>']
        self.eos_token = '<|im_end|>'
        self.pad_token = '<|pad|>'
        self.all_special_tokens = [t for t in self.SPECIAL if t.startswith('<|')]

    def __len__(self):
        return self.vocab_size

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out: List[int] = []
        i = 0
        while i < len(text):
            hit = None
            if text[i] == '<':
                for tok, tid in self.special.items():
                    if text.startswith(tok, i):
                        hit = (tok, tid)
                        break
            if hit:
                out.append(hit[1])
                i += len(hit[0])
            else:
                out.extend(text[i].encode('utf-8'))
                i += 1
        return out

    def __call__(self, text, add_special_tokens=False, **kw):
        if isinstance(text, str):
            return {'input_ids': self.encode(text)}
        return {'input_ids': [self.encode(t) for t in text]}

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        buf, parts = bytearray(), []
        for t in ids:
            t = int(t)
            if t < 256:
                buf.append(t)
            else:
                if buf:
                    parts.append(buf.decode('utf-8', errors='replace'))
                    buf = bytearray()
                # like the Qwen tokenizers: <tool_call> / <think> are single tokens but ordinary text, only control tokens are skipped
                if t in self.inv and (not skip_special_tokens or not self.inv[t].startswith('<|')):
                    parts.append(self.inv[t])
        if buf:
            parts.append(buf.decode('utf-8', errors='replace'))
        return ''.join(parts)

    def convert_tokens_to_ids(self, tok: str) -> int:
        return self.special.get(tok, -1)

    def apply_chat_template(self, messages: List[Dict[str, Any]], tools=None, tokenize: bool = False,
                            add_generation_prompt: bool = False, **kw) -> str:
        s = ''
        if tools:
            s += '<|im_start|>system\n# Tools\n' + '\n'.join(json.dumps(t, ensure_ascii=False) for t in tools) + '<|im_end|>\n'
        for m in messages:
            content = m.get('content') or ''
            if not isinstance(content, str):
                content = ''.join(p.get('text', '') for p in content if isinstance(p, dict))
            if m.get('reasoning_content'):
                content = f"<think>\n{m['reasoning_content']}\n</think>\n\n{content}"
            for tc in m.get('tool_calls') or []:
                args = tc.get('arguments')
                args = args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)
                content += f'\n<tool_call>\n{{"name": "{tc.get("tool_name")}", "arguments": {args}}}\n</tool_call>'
            s += f"<|im_start|>{m['role']}\n{content}<|im_end|>\n"
        if add_generation_prompt:
            s += '<|im_start|>assistant\n'
        return s if not tokenize else self.encode(s)

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, 'byte_chat_tokenizer.json'), 'w') as f:
            json.dump({'type': 'ByteChatTokenizer', 'vocab_size': self.vocab_size}, f)


def load_tokenizer(model_id: Optional[str], vocab_size: int = 1024):
    if model_id and os.path.isdir(str(model_id)) and any(
            os.path.isfile(os.path.join(model_id, f)) for f in ('tokenizer.json', 'tokenizer_config.json', 'vocab.json')):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(model_id, trust_remote_code=False)
    return ByteChatTokenizer(vocab_size)


class Template:
    """``truncation_strategy``: ``raise`` | ``left`` | ``right`` | ``split`` | ``delete``."""

    def __init__(self, model_id: Optional[str] = None, tokenizer=None, max_length: Optional[int] = 8192,
                 truncation_strategy: str = 'raise', default_system: Optional[str] = None, enable_thinking: bool = True,
                 use_chat_template: bool = True, agent_template: Optional[str] = None, **kwargs):
        self.model_id = model_id
        self.tokenizer = tokenizer if tokenizer is not None else load_tokenizer(model_id, kwargs.get('vocab_size', 1024))
        self.max_length = max_length
        self.truncation_strategy = truncation_strategy
        self.default_system = default_system
        self.enable_thinking = enable_thinking
        self.use_chat_template = use_chat_template
        self.agent_template = agent_template
        self.pre_pipeline = [self._add_default_system, self._to_standard_reasoning_content, self._build_standard_messages]
        self.post_pipeline = [self._check_max_length, self._add_attention_fields, self._roll_labels]

    # -------------------------------------------------------- pre-pipeline
    def _add_default_system(self, traj: Trajectory) -> Trajectory:
        msgs = traj.get('messages') or []
        if self.default_system and (not msgs or msgs[0].get('role') != 'system'):
            traj['messages'] = [{'role': 'system', 'content': self.default_system}] + list(msgs)
        return traj

    def _to_standard_reasoning_content(self, traj: Trajectory) -> Trajectory:
        """``<think>…</think>`` inside assistant content moves to ``reasoning_content``."""
        for m in traj.get('messages') or []:
            c = m.get('content')
            # only a block that opens the content counts: a stray closing tag in the middle of an answer stays content, and
            # everything after the FIRST closing tag is kept (later stray tags included), so rendering round-trips
            if (m.get('role') == 'assistant' and isinstance(c, str) and c.lstrip().startswith('<think>') and '</think>' in c
                    and not m.get('reasoning_content')):
                head, tail = c.split('</think>', 1)
                m['reasoning_content'] = head.split('<think>', 1)[1].strip()
                m['content'] = tail.lstrip('\n')
        return traj

    def _build_standard_messages(self, traj: Trajectory) -> Trajectory:
        if not traj.get('messages') and traj.get('prompt'):
            traj['messages'] = [{'role': 'user', 'content': traj['prompt']}]
        for m in traj.get('messages') or []:
            if m.get('content') is None:
                m['content'] = ''
        return traj

    # ------------------------------------------------------------ rendering
    def _render(self, messages: List[Message], tools=None, add_generation_prompt: bool = False) -> List[int]:
        kw = {}
        try:
            text = self.tokenizer.apply_chat_template(messages, tools=tools or None, tokenize=False,
                                                      add_generation_prompt=add_generation_prompt,
                                                      enable_thinking=self.enable_thinking)
        except TypeError:
            text = self.tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt)
        enc = self.tokenizer(text, add_special_tokens=False)
        return list(enc['input_ids'])

    def _encode_rounds(self, messages: List[Message], tools=None) -> Tuple[List[int], List[int]]:
        """Token ids and un-rolled labels: tokenise growing prefixes; tokens added
        by an assistant message (minus the generation prompt) carry labels."""
        ids: List[int] = []
        labels: List[int] = []
        prev: List[int] = []
        for i, m in enumerate(messages):
            if m.get('role') == 'assistant':
                with_prompt = self._render(messages[:i], tools, add_generation_prompt=True) if i > 0 else []
                cur = self._render(messages[:i + 1], tools)
                # common-prefix guard: some chat templates rewrite earlier turns
                k = 0
                while k < min(len(prev), len(cur)) and prev[k] == cur[k]:
                    k += 1
                if k < len(prev):
                    ids, labels = ids[:k], labels[:k]
                new = cur[len(ids):]
                n_prompt = max(0, min(len(with_prompt), len(cur)) - len(ids))
                train = m.get('loss', True) is not False
                ids += new
                labels += [IGNORE] * n_prompt + (list(new[n_prompt:]) if train else [IGNORE] * (len(new) - n_prompt))
                prev = cur
            elif i == len(messages) - 1 or messages[i + 1].get('role') == 'assistant':
                cur = self._render(messages[:i + 1], tools)
                k = 0
                while k < min(len(prev), len(cur)) and prev[k] == cur[k]:
                    k += 1
                if k < len(prev):
                    ids, labels = ids[:k], labels[:k]
                new = cur[len(ids):]
                ids += new
                labels += [IGNORE] * len(new)
                prev = cur
        return ids, labels

    # -------------------------------------------------------- post-pipeline
    def _check_max_length(self, feats: List[InputFeature]) -> List[InputFeature]:
        if not self.max_length:
            return feats
        out = []
        for f in feats:
            n = len(f['input_ids'])
            if n <= self.max_length:
                out.append(f)
                continue
            s = self.truncation_strategy
            if s == 'raise':
                raise ValueError(f'sequence of {n} tokens exceeds max_length={self.max_length}')
            if s == 'delete':
                continue
            if s == 'left':
                out.append({**f, 'input_ids': f['input_ids'][-self.max_length:], 'labels': f['labels'][-self.max_length:]})
            elif s == 'right':
                out.append({**f, 'input_ids': f['input_ids'][:self.max_length], 'labels': f['labels'][:self.max_length]})
            elif s == 'split':
                for a in range(0, n, self.max_length):
                    out.append({**f, 'input_ids': f['input_ids'][a:a + self.max_length], 'labels': f['labels'][a:a + self.max_length]})
            else:
                raise ValueError(f'unknown truncation_strategy {s}')
        return out

    def _add_attention_fields(self, feats: List[InputFeature]) -> List[InputFeature]:
        for f in feats:
            n = len(f['input_ids'])
            f['attention_mask'] = [1] * n
            f['position_ids'] = list(range(n))
            f['length'] = n
        return feats

    @staticmethod
    def _roll_labels(feats: List[InputFeature]) -> List[InputFeature]:
        for f in feats:
            lab = list(f['labels'])
            f['labels'] = lab[1:] + [IGNORE]
        return feats

    # ---------------------------------------------------------------- API
    def encode(self, trajectory: Trajectory, add_generation_prompt: bool = False) -> Union[InputFeature, List[InputFeature]]:
        traj = copy.deepcopy(dict(trajectory))
        for fn in self.pre_pipeline:
            traj = fn(traj)
        msgs = traj.get('messages') or []
        if add_generation_prompt or not any(m.get('role') == 'assistant' for m in msgs):
            ids = self._render(msgs, traj.get('tools'), add_generation_prompt=True)
            labels = [IGNORE] * len(ids)
        else:
            ids, labels = self._encode_rounds(msgs, traj.get('tools'))
        feats: List[InputFeature] = [{'input_ids': ids, 'labels': labels}]
        for fn in self.post_pipeline:
            feats = fn(feats)
        for f in feats:
            if traj.get('user_data') is not None:
                f['user_data'] = traj['user_data']  # type: ignore[typeddict-unknown-key]
        if not feats:
            return []
        return feats[0] if len(feats) == 1 else feats

    def batch_encode(self, trajectories: Sequence[Trajectory], add_generation_prompt: bool = False) -> List[InputFeature]:
        out: List[InputFeature] = []
        for t in trajectories:
            r = self.encode(t, add_generation_prompt)
            out.extend(r if isinstance(r, list) else [r])
        return out

    def decode(self, token_ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(list(token_ids), skip_special_tokens=skip_special_tokens)

    def batch_decode(self, batch: Sequence[Sequence[int]], skip_special_tokens: bool = True) -> List[str]:
        return [self.decode(x, skip_special_tokens) for x in batch]

    @staticmethod
    def concat_input_feature(prompt: InputFeature, new_tokens: Sequence[int]) -> InputFeature:
        """Prompt ⊕ sampled tokens. (Rolled) labels are added on the sampled part — ``labels[t] = input_ids[t+1]`` for
        positions whose next token was sampled — and the prompt keeps the labels it came with, so a feature that is
        extended turn after turn in a multi-turn rollout ends up with every sampled token as a target."""
        p = [int(t) for t in prompt['input_ids']]
        new = [int(t) for t in new_tokens]
        ids = p + new
        old = prompt.get('labels')
        old = [int(x) for x in old] if old is not None and len(old) == len(p) else [IGNORE] * len(p)
        labels = old + [IGNORE] * len(new)
        for t in range(len(p) - 1, len(ids) - 1):
            labels[t] = ids[t + 1]
        n = len(ids)
        out = {'input_ids': ids, 'labels': labels, 'attention_mask': [1] * n, 'position_ids': list(range(n)), 'length': n}
        if prompt.get('pixel_values') is not None:  # images stay with the feature; sampled text continues all three position rows
            import torch
            m = torch.as_tensor(prompt['mrope_position_ids']).long()
            nxt = int(m.max()) + 1 if m.numel() else 0
            out.update(pixel_values=prompt['pixel_values'], image_grid_thw=prompt['image_grid_thw'],
                       mrope_position_ids=torch.cat([m, torch.arange(nxt, nxt + len(new)).expand(3, -1)], 1))
            if prompt.get('placeholder_ids') is not None:
                out['placeholder_ids'] = prompt['placeholder_ids']
        return out

    # ------------------------------------------------------------ tool calls
    def _tool_formats(self):
        return (self.agent_template, ) if self.agent_template else ('hermes', 'vcp', 'react', 'cline')

    def parse_tool_call(self, text: str, known_tools: Optional[Sequence[str]] = None) -> List[Dict[str, Any]]:
        """Tool calls written in a completion, in the template's ``agent_template`` syntax (``hermes`` / ``react`` /
        ``cline`` / ``vcp``) or, when none is set, in the first syntax that matches. Empty list when there is none."""
        from .tools import parse_tool_calls
        return parse_tool_calls(text or '', self._tool_formats(), known_tools=known_tools)[0]

    def clean_tool_call(self, text: str, known_tools: Optional[Sequence[str]] = None) -> str:
        """The completion without its tool-call syntax (what goes into the assistant message's ``content``)."""
        from .tools import parse_tool_calls
        return parse_tool_calls(text or '', self._tool_formats(), known_tools=known_tools)[1]

    def response_message(self, text: str) -> Dict[str, Any]:
        """Assistant message for a decoded completion: content with the call syntax removed, ``tool_calls`` when any."""
        calls = self.parse_tool_call(text)
        msg: Dict[str, Any] = {'role': 'assistant', 'content': self.clean_tool_call(text) if calls else (text or '')}
        if calls:
            msg['tool_calls'] = calls
        return msg

    def pre_forward_hook(self, inputs: Dict[str, Any]) -> Dict[str, Any]:
        """Multimodal templates merge vision embeddings here; text models pass through."""
        return inputs

    @property
    def eos_token_id(self) -> Optional[int]:
        return getattr(self.tokenizer, 'eos_token_id', None)


class Qwen3Template(Template):
    pass


class DeepseekV4Template(Template):
    pass


class Qwen2VLTemplate(Template):
    """Chat template for the Qwen2-VL family: images given as content parts (``{'type': 'image', 'image': path | URL | bytes |
    PIL | array}``) or as ``trajectory['images']`` matched to ``<image>`` markers in the text become
    ``<|vision_start|><|image_pad|>…<|vision_end|>`` with one pad token per merged patch. The encoded feature carries
    ``pixel_values`` (flat patches of all images), ``image_grid_thw`` and ``mrope_position_ids`` ``[3, L]`` (time / height
    / width positions); ``position_ids`` stays the plain token index. Truncation that would cut through an image raises.

    ``vision_config`` is the tower's config (a ``models.vision.VisionConfig`` or its dict); ``min_pixels`` / ``max_pixels``
    bound the resized image. Reference: ``template/base.py:611-667`` + the HF processor it delegates to."""

    IMAGE_MARK = '<|vision_start|><|image_pad|><|vision_end|>'
    VIDEO_MARK = '<|vision_start|><|video_pad|><|vision_end|>'

    def __init__(self, *a, vision_config=None, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280, **kw):
        super().__init__(*a, **kw)
        from ..models.vision import VisionConfig
        self.vision_config = vision_config if isinstance(vision_config, VisionConfig) else VisionConfig.from_hf(dict(vision_config or {}))
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.image_token_id = self.tokenizer.convert_tokens_to_ids('<|image_pad|>')
        self.video_token_id = self.tokenizer.convert_tokens_to_ids('<|video_pad|>')
        self._vision: List[Tuple[Any, Tuple[int, int, int]]] = []
        self.pre_pipeline = self.pre_pipeline + [self._collect_images]
        self.post_pipeline = self.post_pipeline + [self._attach_vision]

    def _collect_images(self, traj: Trajectory) -> Trajectory:
        from ..models.vision import preprocess_image, preprocess_video
        loose = list(traj.get('images') or [])
        sources: List[Any] = []                    # an image source, or ('video', [frames]) for a video part
        for m in traj.get('messages') or []:
            c = m.get('content')
            if isinstance(c, list):
                text = ''
                for part in c:
                    if part.get('type') in ('image', 'image_url'):
                        src = part.get('image', part.get('image_url'))
                        sources.append(src.get('url') if isinstance(src, dict) else src)
                        text += self.IMAGE_MARK
                    elif part.get('type') == 'video':      # a list of frames (decoding video files is left to the caller)
                        sources.append(('video', list(part['video']), part.get('fps')))   # fps: sampled frames per second, if known
                        text += self.VIDEO_MARK
                    else:
                        text += part.get('text', '')
                m['content'] = text
            elif isinstance(c, str) and '<image>' in c:
                for _ in range(c.count('<image>')):
                    if not loose:
                        raise ValueError('more <image> markers than entries in trajectory["images"]')
                    sources.append(loose.pop(0))
                m['content'] = c.replace('<image>', self.IMAGE_MARK)
        if loose:  # images without a marker go in front of the first user turn, in order
            first = next((m for m in traj.get('messages') or [] if m.get('role') == 'user'), None)
            if first is None:
                raise ValueError('trajectory["images"] given but there is no user message to attach them to')
            n_before = sum(str(m.get('content', '')).count(self.IMAGE_MARK) for m in traj['messages'][:traj['messages'].index(first)])
            first['content'] = self.IMAGE_MARK * len(loose) + str(first.get('content') or '')
            sources[n_before:n_before] = loose
        vc = self.vision_config
        # Qwen2.5-VL lays video frames out in real time: one temporal patch spans temporal_patch_size / fps seconds
        self._time_steps = [(vc.temporal_patch_size / float(src[2]) * vc.tokens_per_second if vc.arch == 'qwen2_5_vl' and isinstance(src, tuple)
                             and len(src) == 3 and src[0] == 'video' and src[2] else None) for src in sources]
        self._vision = [preprocess_video(src[1], self.vision_config) if isinstance(src, tuple) and len(src) == 3 and src[0] == 'video'
                        else preprocess_image(src, self.vision_config, self.min_pixels, self.max_pixels) for src in sources]
        return traj

    def _render(self, messages, tools=None, add_generation_prompt: bool = False) -> List[int]:
        ids = super()._render(messages, tools, add_generation_prompt)
        if not self._vision:
            return ids
        merge2 = self.vision_config.spatial_merge_size**2
        out, k = [], 0
        for t in ids:
            if t in (self.image_token_id, self.video_token_id) and k < len(self._vision):
                g = self._vision[k][1]
                out.extend([t] * (g[0] * g[1] * g[2] // merge2))
                k += 1
            else:
                out.append(t)
        return out

    def _attach_vision(self, feats: List[InputFeature]) -> List[InputFeature]:
        if not self._vision:
            return feats
        import torch
        from ..models.vision import rope_index
        if len(feats) != 1:
            raise ValueError('a trajectory with images cannot be split into several features; raise max_length')
        f = feats[0]
        grids = [g for _, g in self._vision]
        f['pixel_values'] = torch.cat([p for p, _ in self._vision], 0)                      # type: ignore[typeddict-unknown-key]
        f['placeholder_ids'] = [self.image_token_id, self.video_token_id]                   # type: ignore[typeddict-unknown-key]
        f['image_grid_thw'] = [list(g) for g in grids]                                      # type: ignore[typeddict-unknown-key]
        f['mrope_position_ids'] = rope_index(f['input_ids'], grids, self.image_token_id,   # type: ignore[typeddict-unknown-key]
                                             self.vision_config.spatial_merge_size, video_token_id=self.video_token_id,
                                             time_steps=getattr(self, '_time_steps', None))
        return feats


class Qwen3_5Template(Qwen2VLTemplate):
    """Qwen3.5: the hybrid-thinking chat format (an empty ``<think>`` block is emitted when thinking is disabled, so that the
    label mask matches generation) with the family's image and video parts (reference ``template/qwen3_5_vl.py:33-200``, where
    the one class serves text and vision-language checkpoints alike).  Without ``vision_config`` — a text-only checkpoint —
    it is a plain chat template; a trajectory that carries images then fails in the tower-less model, not here."""

    def __init__(self, *a, enable_thinking: bool = True, vision_config=None, **kw):
        super().__init__(*a, enable_thinking=enable_thinking, vision_config=vision_config, **kw)


template_mapping = {'Template': Template, 'default': Template, 'Qwen3Template': Qwen3Template, 'qwen3': Qwen3Template,
                    'Qwen3_5Template': Qwen3_5Template, 'qwen3_5': Qwen3_5Template, 'DeepseekV4Template': DeepseekV4Template,
                    'Qwen2VLTemplate': Qwen2VLTemplate, 'qwen2_vl': Qwen2VLTemplate, 'Qwen3VLTemplate': Qwen2VLTemplate, 'qwen3_vl': Qwen2VLTemplate,
                    'Qwen3_5VLTemplate': Qwen3_5Template, 'qwen3_5_vl': Qwen3_5Template}
