"""Client of a Search-R1 style retrieval service (verl/tools/utils/search_r1_like_utils.py:34-250).

``call_search_api`` POSTs ``{"queries", "topk", "return_scores"}`` and retries on 5xx answers, connection errors
and timeouts with a growing delay; ``perform_single_search_batch`` formats the passages the way the Search-R1
prompts expect and returns (JSON text for the model, metadata for logging)."""

from __future__ import annotations

import json
import logging
import threading
import time
import uuid
from typing import Any, Optional

logger = logging.getLogger(__name__)

DEFAULT_TIMEOUT = 30
MAX_RETRIES = 10
INITIAL_RETRY_DELAY = 1.0
RETRY_STATUS = (500, 502, 503, 504)


def call_search_api(retrieval_service_url: str, query_list: list[str], topk: int = 3, return_scores: bool = True,
                    timeout: int = DEFAULT_TIMEOUT, max_retries: int = MAX_RETRIES,
                    retry_delay: float = INITIAL_RETRY_DELAY) -> tuple[Optional[dict[str, Any]], Optional[str]]:
    """Returns (response json, None) or (None, error text) after ``max_retries`` attempts."""
    import requests

    rid = uuid.uuid4().hex[:8]
    payload = {"queries": query_list, "topk": topk, "return_scores": return_scores}
    last = None
    for attempt in range(max_retries):
        try:
            r = requests.post(retrieval_service_url, json=payload, timeout=timeout,
                              headers={"Content-Type": "application/json", "Accept": "application/json"})
            if r.status_code in RETRY_STATUS:
                last = f"API Request Error: server answered {r.status_code}"
            else:
                r.raise_for_status()
                return r.json(), None
        except requests.exceptions.ConnectionError as e:
            last = f"Connection Error: {e}"
        except requests.exceptions.Timeout as e:
            last = f"Timeout Error: {e}"
        except requests.exceptions.RequestException as e:  # 4xx and the like: retrying will not help
            return None, f"API Request Error: {e}"
        except json.JSONDecodeError as e:
            return None, f"API Response JSON Decode Error: {e}"
        logger.warning("[Search Request ID: %s] %s (attempt %d of %d)", rid, last, attempt + 1, max_retries)
        if attempt + 1 < max_retries:
            time.sleep(retry_delay * (attempt + 1))
    return None, (last or "API Request Error: unknown").replace("API Request Error", "API Request Error after retries")


def _passages2string(retrieval_result: list[dict]) -> str:
    out = []
    for i, doc in enumerate(retrieval_result):
        content = doc.get("document", {}).get("contents", "") if isinstance(doc.get("document"), dict) else str(doc)
        title, _, text = content.partition("\n")
        out.append(f"Doc {i + 1} (Title: {title})\n{text}\n")
    return "\n".join(out)


def perform_single_search_batch(retrieval_service_url: str, query_list: list[str], topk: int = 3,
                                concurrent_semaphore: Optional[threading.Semaphore] = None, timeout: int = DEFAULT_TIMEOUT,
                                **retry_kwargs) -> tuple[str, dict[str, Any]]:
    meta = {"query_count": len(query_list), "queries": query_list, "api_request_error": None, "api_response": None,
            "status": "unknown", "total_results": 0, "formatted_result": None}
    try:
        if concurrent_semaphore is not None:
            with concurrent_semaphore:
                resp, err = call_search_api(retrieval_service_url, query_list, topk, True, timeout, **retry_kwargs)
        else:
            resp, err = call_search_api(retrieval_service_url, query_list, topk, True, timeout, **retry_kwargs)
    except Exception as e:
        resp, err = None, f"API Request Exception during batch search: {e}"
    meta["api_request_error"], meta["api_response"] = err, resp
    if err:
        text = json.dumps({"result": f"Search error: {err}"}, ensure_ascii=False)
        meta["status"] = "api_error"
    elif resp:
        results = resp.get("result", [])
        if results:
            pretty = "\n---\n".join(_passages2string(x) for x in results)
            meta["total_results"] = sum(len(x) for x in results if isinstance(x, list))
            meta["status"], meta["formatted_result"] = "success", pretty
            text = json.dumps({"result": pretty}, ensure_ascii=False)
        else:
            text = json.dumps({"result": "No search results found."}, ensure_ascii=False)
            meta["status"] = "no_results"
    else:
        text = json.dumps({"result": "Search request failed or timed out after retries."}, ensure_ascii=False)
        meta["status"] = "unknown_api_state"
    return text, meta
