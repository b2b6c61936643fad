"""Model name -> provider routing and one ``generate_code`` entry point.

Eight providers, as in the reference's ``prompt_llm/llm_factory.py`` (provider enum :11-20,
model table :24-89, prefix routing :92-142, ``generate_code`` :183-233,
``list_supported_models`` :236-256) and its per-provider clients (``gpt.py``,
``anthropic_llm.py``, ``gemini.py``, ``grok.py``, ``deepseek.py``, ``glm.py``, ``qwen.py``,
``moonshot.py``).  Here every provider is a small description (endpoint, key variables, wire
format, quirks) run by one HTTP client built on the standard library, so no vendor SDK is
needed; tests inject a fake transport, and the GPU machines (no network) never call out.
"""
from __future__ import annotations

import json
import os
import random
import time
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from enum import Enum

from .prompt import extract_code_from_response

SYSTEM_MESSAGE = ("You are an expert programmer of GPU communication software (CUDA, NCCL, RDMA). "
                  "You answer with complete, compilable source files.")


class Provider(str, Enum):
    OPENAI = "openai"
    ANTHROPIC = "anthropic"
    GEMINI = "gemini"
    GROK = "grok"
    DEEPSEEK = "deepseek"
    GLM = "glm"
    QWEN = "qwen"
    MOONSHOT = "moonshot"


@dataclass
class ProviderSpec:
    provider: Provider
    url: str
    key_env: tuple[str, ...]
    wire: str = "openai"                      # "openai" (chat completions), "anthropic", "gemini"
    models: tuple[str, ...] = ()
    prefixes: tuple[str, ...] = ()
    timeout_env: str = "LLM_HTTP_TIMEOUT"
    extra_headers: dict = field(default_factory=dict)


SPECS: dict[Provider, ProviderSpec] = {
    Provider.OPENAI: ProviderSpec(
        Provider.OPENAI, "https://api.openai.com/v1/chat/completions", ("OPENAI_API_KEY",),
        models=("gpt-4o", "gpt-4o-mini", "gpt-4-turbo", "gpt-4", "gpt-3.5-turbo", "o1", "o1-mini",
                "o1-preview", "o3-mini", "gpt-5", "gpt-5.2"),
        prefixes=("gpt", "o1", "o3", "o4"), timeout_env="OPENAI_HTTP_TIMEOUT"),
    Provider.ANTHROPIC: ProviderSpec(
        Provider.ANTHROPIC, "https://api.anthropic.com/v1/messages", ("ANTHROPIC_API_KEY",),
        wire="anthropic", models=("claude-3-5-sonnet-latest", "claude-3-opus-latest",
                                  "claude-sonnet-4-5", "claude-opus-4-5"),
        prefixes=("claude",), extra_headers={"anthropic-version": "2023-06-01"}),
    Provider.GEMINI: ProviderSpec(
        Provider.GEMINI, "https://generativelanguage.googleapis.com/v1beta/models/{model}:generateContent",
        ("GOOGLE_API_KEY", "GEMINI_API_KEY"), wire="gemini",
        models=("gemini-1.5-pro", "gemini-1.5-flash", "gemini-2.0-flash", "gemini-2.5-pro",
                "gemini-3-pro-preview"), prefixes=("gemini",)),
    Provider.GROK: ProviderSpec(
        Provider.GROK, "https://api.x.ai/v1/chat/completions", ("XAI_API_KEY", "GROK_API_KEY"),
        models=("grok-2", "grok-3", "grok-4"), prefixes=("grok",)),
    Provider.DEEPSEEK: ProviderSpec(
        Provider.DEEPSEEK, "https://api.deepseek.com/chat/completions", ("DEEPSEEK_API_KEY",),
        models=("deepseek-chat", "deepseek-reasoner"), prefixes=("deepseek",)),
    Provider.GLM: ProviderSpec(
        Provider.GLM, "https://open.bigmodel.cn/api/paas/v4/chat/completions", ("GLM_API_KEY",),
        models=("glm-4", "glm-4.6"), prefixes=("glm", "z-ai/glm")),
    Provider.QWEN: ProviderSpec(
        Provider.QWEN, "https://dashscope.aliyuncs.com/compatible-mode/v1/chat/completions",
        ("QWEN_API_KEY", "DASHSCOPE_API_KEY"), models=("qwen-max", "qwen3-coder-plus", "qwen3-max"),
        prefixes=("qwen",)),
    Provider.MOONSHOT: ProviderSpec(
        Provider.MOONSHOT, "https://api.moonshot.cn/v1/chat/completions", ("MOONSHOT_API_KEY",),
        models=("moonshot-v1-128k", "kimi-k2-0905-preview", "kimi-k2-thinking"),
        prefixes=("kimi", "moonshot")),
}


class LLMError(RuntimeError):
    def __init__(self, msg: str, status: int | None = None, transient: bool = False):
        super().__init__(msg)
        self.status, self.transient = status, transient


def provider_for_model(model: str) -> Provider:
    m = model.lower()
    for spec in SPECS.values():
        if m in spec.models:
            return spec.provider
    for spec in SPECS.values():
        if any(m.startswith(p) for p in spec.prefixes):
            return spec.provider
    raise LLMError(f"no provider known for model {model!r}")


def list_supported_models() -> dict[str, list[str]]:
    return {s.provider.value: list(s.models) for s in SPECS.values()}


def is_reasoning_model(model: str) -> bool:
    """Models that pick their own sampling settings and reject ``temperature``."""
    m = model.lower()
    return (m.startswith(("o1", "o3", "o4", "gpt-5")) or m == "deepseek-reasoner"
            or "thinking" in m)


def build_request(spec: ProviderSpec, model: str, prompt: str, temperature: float | None,
                  api_key: str, max_tokens: int = 16384) -> tuple[str, dict, dict]:
    """(url, headers, body) for one completion.  Per-provider quirks live here."""
    headers = {"Content-Type": "application/json", **spec.extra_headers}
    m = model.lower()
    if spec.wire == "anthropic":
        headers["x-api-key"] = api_key
        body = {"model": model, "max_tokens": max_tokens, "system": SYSTEM_MESSAGE,
                "messages": [{"role": "user", "content": prompt}]}
        if temperature is not None and "thinking" not in m:
            body["temperature"] = temperature
        return spec.url, headers, body
    if spec.wire == "gemini":
        body = {"systemInstruction": {"parts": [{"text": SYSTEM_MESSAGE}]},
                "contents": [{"role": "user", "parts": [{"text": prompt}]}],
                "generationConfig": {"maxOutputTokens": max_tokens}}
        if temperature is not None:
            body["generationConfig"]["temperature"] = temperature
        return spec.url.format(model=model) + f"?key={api_key}", headers, body
    headers["Authorization"] = f"Bearer {api_key}"
    body = {"model": model, "messages": [{"role": "system", "content": SYSTEM_MESSAGE},
                                          {"role": "user", "content": prompt}]}
    if spec.provider is Provider.OPENAI and is_reasoning_model(model):
        body["max_completion_tokens"] = max_tokens         # these reject temperature / max_tokens
    else:
        body["max_tokens"] = max_tokens
        if temperature is not None and not is_reasoning_model(model):
            body["temperature"] = temperature
    if spec.provider is Provider.MOONSHOT and m.startswith("kimi-k2"):
        body["temperature"] = 1.0                           # the only value these accept
    if spec.provider is Provider.QWEN and m.startswith("qwen3"):
        body["enable_thinking"] = False                     # non-streaming calls require it off
    return spec.url, headers, body


def parse_reply(spec: ProviderSpec, payload: dict) -> str:
    try:
        if spec.wire == "anthropic":
            return "".join(b.get("text", "") for b in payload["content"] if b.get("type") == "text")
        if spec.wire == "gemini":
            return "".join(p.get("text", "") for p in payload["candidates"][0]["content"]["parts"])
        return payload["choices"][0]["message"]["content"] or ""
    except (KeyError, IndexError, TypeError) as e:
        raise LLMError(f"unexpected reply shape from {spec.provider.value}: {e}") from e


def _http_post(url: str, headers: dict, body: dict, timeout: float) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers=headers, method="POST")
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            return json.loads(r.read().decode())
    except urllib.error.HTTPError as e:
        transient = e.code in (408, 409, 425, 429) or e.code >= 500
        raise LLMError(f"HTTP {e.code}: {e.read()[:300]!r}", e.code, transient) from e
    except (urllib.error.URLError, TimeoutError, ConnectionError) as e:
        raise LLMError(f"network error: {e}", None, True) from e


def is_transient(err: Exception) -> bool:
    if isinstance(err, LLMError):
        return err.transient
    text = str(err).lower()
    return any(k in text for k in ("timeout", "timed out", "rate limit", "overloaded", "temporarily",
                                   "connection reset", "503", "502", "429"))


def backoff_delay(attempt: int, base: float = 2.0, cap: float = 60.0, rng=random.random) -> float:
    """``base * 2^attempt`` plus up to one ``base`` of jitter, capped."""
    return min(cap, base * (2 ** attempt) + rng() * base)


def generate_response(prompt: str, model: str, temperature: float | None = 0.2,
                      api_key: str | None = None, transport=None, max_retries: int | None = None,
                      sleep=time.sleep) -> str:
    """Raw text of one completion, with retries on transient failures.  ``transport`` replaces
    the HTTP POST (``transport(url, headers, body, timeout) -> dict``)."""
    spec = SPECS[provider_for_model(model)]
    key = api_key or next((os.environ[k] for k in spec.key_env if os.environ.get(k)), None)
    if not key:
        raise LLMError(f"no API key: set {' or '.join(spec.key_env)}")
    url, headers, body = build_request(spec, model, prompt, temperature, key)
    timeout = float(os.environ.get(spec.timeout_env, os.environ.get("LLM_HTTP_TIMEOUT", "600")))
    retries = int(os.environ.get("LLM_MAX_RETRIES", "3")) if max_retries is None else max_retries
    post = transport or _http_post
    for attempt in range(retries + 1):
        try:
            return parse_reply(spec, post(url, headers, body, timeout))
        except Exception as e:               # noqa: BLE001 - classified below
            if attempt == retries or not is_transient(e):
                raise
            sleep(backoff_delay(attempt))
    raise AssertionError("unreachable")


def generate_code(prompt: str, model: str, language: str = "cuda", temperature: float | None = 0.2,
                  api_key: str | None = None, transport=None, **kw) -> str:
    """One completion reduced to the program it contains."""
    return extract_code_from_response(
        generate_response(prompt, model, temperature, api_key, transport, **kw), language)
