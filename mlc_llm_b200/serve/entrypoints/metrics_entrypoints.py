"""``GET /metrics``: engine metrics as Prometheus text (reference:
``python/mlc_llm/serve/entrypoints/metrics_entrypoints.py:13-23``)."""

import fastapi
from fastapi.responses import PlainTextResponse

from ..server.server_context import ServerContext

app = fastapi.APIRouter()


@app.get("/metrics", response_class=PlainTextResponse)
async def metrics(_request: fastapi.Request):
    ctx = ServerContext.current()
    parts = []
    for model in ctx.get_model_list():
        engine = ctx.get_engine(model)
        if engine is None or not hasattr(engine, "metrics"):
            continue
        parts.append((await engine.metrics()).prometheus_text())
    return "\n".join(parts)
