// Command-line front end with the reference binary's arguments and output protocol
// (src/bin/engine_gpt2.rs:8): brrr_engine <data-dir> <blob> [prompt|--serve] [ngen].
#include "../../include/brrr.h"

int main(int argc, char **argv) { return brrr_cli_main(argc, argv); }
