"""Error bodies returned by the REST server (reference: ``protocol/error_protocol.py``)."""
from http import HTTPStatus
from typing import Optional

import fastapi
from pydantic import BaseModel


class BadRequestError(ValueError):
    """Invalid request content; rendered as HTTP 400."""


class RequestFailedError(RuntimeError):
    """The engine could not finish a request (a step raised); rendered as HTTP 500."""


class ErrorResponse(BaseModel):
    object: str = "error"
    message: str
    code: Optional[int] = None


def create_error_response(status_code: HTTPStatus, message: str) -> fastapi.responses.JSONResponse:
    return fastapi.responses.JSONResponse(
        ErrorResponse(message=message, code=status_code.value).model_dump(by_alias=True),
        status_code=status_code.value,
    )


async def bad_request_error_handler(_request: fastapi.Request, e: BadRequestError):
    return create_error_response(HTTPStatus.BAD_REQUEST, message=e.args[0])
