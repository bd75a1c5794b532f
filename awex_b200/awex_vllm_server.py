"""``python -m awex_b200.awex_vllm_server <vllm serve args>``: vLLM's
OpenAI-compatible server with the Awex routes and worker methods registered
(`awex/awex_vllm_server.py:36-53` in the reference)."""

from __future__ import annotations


def main() -> None:
    import uvloop
    from vllm.entrypoints.openai.api_server import run_server
    from vllm.entrypoints.openai.cli_args import make_arg_parser, validate_parsed_serve_args
    from vllm.entrypoints.utils import cli_env_setup

    try:
        from vllm.utils import FlexibleArgumentParser
    except ImportError:
        from vllm.utils.argparse_utils import FlexibleArgumentParser

    from awex_b200.vllm_plugin import register_awex_routes

    register_awex_routes()
    cli_env_setup()
    parser = make_arg_parser(FlexibleArgumentParser(description="vLLM OpenAI-compatible server with Awex weight-update routes."))
    args = parser.parse_args()
    validate_parsed_serve_args(args)
    uvloop.run(run_server(args))


if __name__ == "__main__":
    main()
