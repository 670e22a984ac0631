#pragma once
#include <string>
#include <string_view>
namespace re2 { using StringPiece = std::string_view;
class RE2 { public: RE2(const std::string&){} static std::string QuoteMeta(const std::string& s){return s;} template<class... A> static bool FindAndConsume(StringPiece*, const RE2&, A...){return false;} }; }
