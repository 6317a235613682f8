#!/bin/sh
# Build the host library's tensor-level C ABI for WebAssembly with Emscripten (emcc on PATH).
# Output: spiraltorch_host.mjs + spiraltorch_host.wasm next to this script.
set -eu
here=$(cd "$(dirname "$0")" && pwd)
root=$(cd "$here/../.." && pwd)
exports=$(node --input-type=module -e 'import {EXPORTED} from "'"$here"'/spiraltorch.mjs"; console.log(["malloc","free",...EXPORTED].map(s=>"_"+s).join(","))')
emcc -O3 -std=c++17 -pthread -sPTHREAD_POOL_SIZE=4 -sWASM_BIGINT -sALLOW_MEMORY_GROWTH -sMODULARIZE -sEXPORT_ES6 \
     -sEXPORTED_FUNCTIONS="$exports" -sEXPORTED_RUNTIME_METHODS=UTF8ToString,HEAPF32,HEAPU32,HEAPU8 \
     -I "$root/include" "$root/csrc/host/tensor_abi.cpp" -o "$here/spiraltorch_host.mjs"
