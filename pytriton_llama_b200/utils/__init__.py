from .prompts import ChatPrompt, Llama3ChatPrompt, PlainPrompt, prompt_for_tokenizer

__all__ = ["ChatPrompt", "Llama3ChatPrompt", "PlainPrompt", "prompt_for_tokenizer"]
