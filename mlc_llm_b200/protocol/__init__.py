"""Wire protocols: OpenAI-style requests/responses, generation / debug configs, conversation
templates and the ``mlc-chat-config.json`` schema."""
