// Command-line front end with the qwen3moe reference binary's arguments and output protocol
// (src/bin/engine_qwen2.rs:486-489, 622-683): brrr_engine_qwen <data-dir> <blob> [prompt|--serve] [ngen].
#include "../../include/brrr.h"

int main(int argc, char **argv) { return brrr_qwen_cli_main(argc, argv); }
