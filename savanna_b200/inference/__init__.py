from .generation import generate, sample_tokens, InferenceParams, stream_tokens, generate_samples_from_prompt

__all__ = ["generate", "sample_tokens", "InferenceParams", "stream_tokens", "generate_samples_from_prompt"]
