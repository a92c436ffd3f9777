"""OpenAI-compatible server: request validation, tokenizer, chat templates, engine thread, HTTP routes, CLI."""
