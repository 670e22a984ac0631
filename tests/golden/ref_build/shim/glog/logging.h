// probe-only shim for glog (not product code)
#pragma once
#include <iostream>
#include <sstream>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <algorithm>
#include <fstream>
namespace shimlog {
struct Msg { bool fatal; std::ostringstream s; Msg(bool f):fatal(f){} ~Msg(){ if(fatal){ std::cerr<<s.str()<<std::endl; std::abort(); } } template<class T> Msg& operator<<(const T& v){ s<<v; return *this;} };
struct Voidify { void operator&(Msg&){} void operator&(std::ostream&){} };
}
#define LOG(sev) ::shimlog::Msg(std::strcmp(#sev,"FATAL")==0)
#define LOG_IF(sev, cond) !(cond) ? (void)0 : ::shimlog::Voidify() & LOG(sev)
#define VLOG(n) if (false) ::shimlog::Msg(false)
#define CHECK(c) (c) ? (void)0 : ::shimlog::Voidify() & ::shimlog::Msg(true) << "CHECK failed: " #c " "
#define CHECK_OP(a,b,op) CHECK((a) op (b))
#define CHECK_EQ(a,b) CHECK_OP(a,b,==)
#define CHECK_NE(a,b) CHECK_OP(a,b,!=)
#define CHECK_GE(a,b) CHECK_OP(a,b,>=)
#define CHECK_GT(a,b) CHECK_OP(a,b,>)
#define CHECK_LE(a,b) CHECK_OP(a,b,<=)
#define CHECK_LT(a,b) CHECK_OP(a,b,<)
namespace google { inline void InitGoogleLogging(const char*){} }
