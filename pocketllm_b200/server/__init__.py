"""OpenAI-compatible serving: request queue, HTTP front end, streaming decoder."""
