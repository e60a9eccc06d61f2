"""Serving front ends: capability manifests, resident models, executor lanes with admission control,
OpenAI / Anthropic / OpenRouter HTTP dialects and the JSONL stdio protocol."""
