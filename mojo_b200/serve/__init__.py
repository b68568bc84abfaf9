"""OpenAI-compatible HTTP server (`/v1/completions`, `/v1/chat/completions`, SSE streaming, `/v1/models`, `/health`,
`/metrics`)."""
from .api_server import AsyncEngine, build_app  # noqa: F401
