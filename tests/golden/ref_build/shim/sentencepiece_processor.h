#pragma once
#include <cstdlib>
#include <string>
#include <vector>
namespace sentencepiece { namespace util { enum class StatusCode { kOk=0 }; struct Status { StatusCode code() const { return StatusCode::kOk; } }; }
class SentencePieceProcessor { public: util::Status Load(const std::string&){return {};} std::vector<int> EncodeAsIds(const std::string&) const {return {};} std::string DecodeIds(const std::vector<int>&) const {return "";} int bos_id() const {return 1;} int eos_id() const {return -7;} int GetPieceSize() const { const char* e=getenv("SHIM_VOCAB"); return e?atoi(e):0; } }; }
