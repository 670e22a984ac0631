// probe-only: stand-ins for op/encode.cpp (needs absl/re2/nlohmann/sentencepiece, absent here)
#include "op/encode.h"
namespace op {
SpeEncodeLayer::SpeEncodeLayer(std::string p, bool b, bool e):EncodeLayerBase(std::move(p),b,e){ spe=std::make_unique<sentencepiece::SentencePieceProcessor>(); }
std::vector<int32_t> SpeEncodeLayer::encode(const std::string&) const { return {1}; }
std::string SpeEncodeLayer::decode(int32_t) const { return ""; }
std::string SpeEncodeLayer::decode(const std::vector<int32_t>&) const { return ""; }
bool SpeEncodeLayer::is_sentence_ending(int32_t t) const { return t==spe->eos_id(); }
int32_t SpeEncodeLayer::vocab_size() const { return spe->GetPieceSize(); }
BpeEncodeLayer::BpeEncodeLayer(std::string p, bool b, bool e):EncodeLayerBase(std::move(p),b,e){}
std::vector<int32_t> BpeEncodeLayer::encode(const std::string&) const { return {1}; }
std::string BpeEncodeLayer::decode(int32_t) const { return ""; }
std::string BpeEncodeLayer::decode(const std::vector<int32_t>&) const { return ""; }
bool BpeEncodeLayer::is_sentence_ending(int32_t) const { return false; }
int32_t BpeEncodeLayer::vocab_size() const { return 0; }
QwenEncodeLayer::QwenEncodeLayer(std::string p, bool b, bool e):BpeEncodeLayer(std::move(p),b,e){}
}
